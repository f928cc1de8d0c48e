"""The reference's OWN device kernels, run unmodified on the GPU, against the CPU oracle and the product kernels.

oracle/build_ref.py compiles the kernel-only prefix of the reference's Inference.cu (the rest of that file does
not compile with this toolkit) behind five C entry points into oracle/_ref/libref_kernels.so; the library is
built where the reference checkout is present and travels with the repository.  These tests pin the oracle:
dequantAwqKernel and applyRotaryKernel must agree with it (and with the product kernels) bit for bit, geluKernel
up to the last bit of erff, rmsNormKernel up to its own fp32 summation order, and the reference's cublasGemmEx call
on the reference's dequantised buffer within the last fp16 bit.  Without the library the tests skip."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from test_gemv_gpu import _run_gemv, _to_dev, _ulp_diff

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "_ref", "libref_kernels.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libref_kernels.so not built (needs the reference checkout at build time)")
    L = C.CDLL(REF_SO)
    vp = C.c_void_p
    L.ref_dequant.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, vp]
    L.ref_rmsnorm.argtypes = [vp, vp, vp, C.c_int, C.c_float, vp]
    L.ref_rotary.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]
    L.ref_gelu.argtypes = [vp, C.c_int, vp]
    L.ref_gemv_cublas.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]
    return L


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


# Shapes on which the reference indexes its scale / zero-point arrays in range (in_dim / 128 <= out_dim / 128
# entries, Inference.cu:90): wqkv / w1, wo, and a slice-sized unembed.  w2 and word_embedding read past their arrays
# in the reference and are covered by the oracle's wrapped index only.
@pytest.mark.parametrize("rows,cols", [(12288, 4096), (4096, 4096), (1536, 512), (9472, 4096)])
def test_reference_dequant_kernel_equals_oracle_and_product(ref, ops, orc, cuda, rows, cols):
    p, s, z = orc.gen_linear(51, rows, cols)
    want = orc.dequant(p, s, z, rows, cols)
    dp, ds, dz = _to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda)
    out = torch.empty((rows, cols), dtype=torch.float16, device=cuda)
    assert ref.ref_dequant(_ptr(dp), _ptr(ds), _ptr(dz), _ptr(out), rows, cols, None) == 0
    torch.cuda.synchronize()
    got_ref = out.cpu().numpy()
    assert np.array_equal(_bits(got_ref), _bits(want)), "oracle differs from the reference's dequantAwqKernel"
    got = ops.dequant_w4(dp, ds, dz, rows, cols).cpu().numpy()
    assert np.array_equal(_bits(got), _bits(got_ref)), "qw3_dequant_w4 differs from the reference's dequantAwqKernel"


def test_reference_dequant_kernel_fractional_zero_points(ref, ops, orc, cuda):
    rows, cols = 1024, 512
    p, s, _ = orc.gen_linear(52, rows, cols)
    z = orc.gen_normal_f16(52, 999, rows // 128, 7.5, 1.3)
    dp, ds, dz = _to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda)
    out = torch.empty((rows, cols), dtype=torch.float16, device=cuda)
    assert ref.ref_dequant(_ptr(dp), _ptr(ds), _ptr(dz), _ptr(out), rows, cols, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(_bits(out.cpu().numpy()), _bits(orc.dequant(p, s, z, rows, cols)))
    assert np.array_equal(_bits(ops.dequant_w4(dp, ds, dz, rows, cols).cpu().numpy()), _bits(out.cpu().numpy()))


def test_reference_rotary_kernel_equals_oracle_and_product(ref, ops, orc, cuda):
    heads, max_pos = 32, 256
    H = heads * 128
    qkv = orc.gen_normal_f16(53, orc.ACT, 3 * H)
    cos_t, sin_t = orc.rope_tables(max_pos, 128, 10000.0)
    dcos, dsin = _to_dev(cos_t, cuda), _to_dev(sin_t, cuda)
    for pos in (0, 1, 100, 255):
        q = _to_dev(qkv[:H].copy(), cuda)
        assert ref.ref_rotary(_ptr(q), _ptr(dcos), _ptr(dsin), heads, 128, pos, None) == 0
        torch.cuda.synchronize()
        got_ref = q.cpu().numpy()
        assert np.array_equal(_bits(got_ref), _bits(orc.rope(qkv[:H], heads, 128, cos_t, sin_t, pos)))
        q2 = torch.zeros(H, dtype=torch.float16, device=cuda)
        kc = torch.zeros(heads, max_pos, 128, dtype=torch.float16, device=cuda)
        vc = torch.zeros_like(kc)
        ops.rope_kv_append(_to_dev(qkv, cuda), q2, kc, vc, dcos, dsin, heads, max_pos, pos)
        assert np.array_equal(_bits(q2.cpu().numpy()), _bits(got_ref))


def test_reference_gelu_kernel_against_oracle(ref, orc, cuda):
    """geluKernel (fp32 erff on the device; the product's GELU epilogue is the same expression on the device) against
    the oracle (erff of the host C library)."""
    x = orc.gen_normal_f16(54, orc.ACT, 12288, 0.0, 2.0)
    d = _to_dev(x.copy(), cuda)
    assert ref.ref_gelu(_ptr(d), x.size, None) == 0
    torch.cuda.synchronize()
    got, want = d.cpu().numpy(), orc.gelu(x)
    diff = _ulp_diff(got, want)
    # device and host erff differ in their last fp32 bit here and there; in the negative tail 1 + erf cancels and
    # that bit becomes a few fp16 ulps of a value that is itself ~1e-3 of the input: compare those on absolute error
    near = np.abs(got.astype(np.float32) - want.astype(np.float32)) <= 3e-4 * np.abs(x.astype(np.float32)).mean()
    frac = float((diff > 0).mean())
    assert ((diff <= 1) | near).all() and frac < 0.02, (int(diff.max()), frac, int((~((diff <= 1) | near)).sum()))


@pytest.mark.parametrize("n", [4096])
def test_reference_rmsnorm_kernel_against_oracle_and_product(ref, ops, orc, cuda, n):
    """The reference sums x^2 in fp32 with a 256-thread tree (Inference.cu:122-135); the oracle and the product sum
    in double.  The fp16-rounded scale can therefore differ in its last bit on rare inputs; where the scales agree
    the outputs must be bit-equal."""
    agree = 0
    for seed in range(8):
        x = orc.gen_normal_f16(60 + seed, orc.ACT, n, 0.0, 3.0)
        g = orc.gen_normal_f16(60 + seed, orc.GAMMA, n, 1.0, 0.02)
        dx, dg = _to_dev(x, cuda), _to_dev(g, cuda)
        out = torch.empty(n, dtype=torch.float16, device=cuda)
        assert ref.ref_rmsnorm(_ptr(dx), _ptr(dg), _ptr(out), n, 1e-6, None) == 0
        torch.cuda.synchronize()
        got_ref, want = out.cpu().numpy(), orc.rmsnorm(x, g)
        got = ops.rmsnorm(dx, dg).cpu().numpy()
        assert np.array_equal(_bits(got), _bits(want))                       # product == oracle, always
        assert _ulp_diff(got_ref, want).max() <= 2                           # a last-bit scale moves outputs by <= 2 ulp
        agree += int(np.array_equal(_bits(got_ref), _bits(want)))
    assert agree >= 6, f"reference rmsNormKernel bit-equal to the oracle on only {agree} of 8 inputs"


@pytest.mark.parametrize("M,K", [(4096, 4096), (12288, 4096), (1536, 512)])
def test_reference_contraction_dequant_then_cublas(ref, ops, orc, cuda, M, K):
    """The reference's contraction, run as the reference runs it: dequantAwqKernel into an fp16 buffer, then
    cublasGemmEx(OP_N, OP_N, m = out_dim, n = 1, k = in_dim, lda = out_dim) on it (Inference.cu:1049-1065).  This pins
    the oracle's reading of the buffer (column-major, element (i, j) at i + j * out_dim) and its fp32 sum; the
    fp16-accumulating compute type is looser by its own rounding and is only bounded."""
    p, s, z = orc.gen_linear(0, M, K)
    x = orc.gen_normal_f16(0, orc.ACT, K)
    y32, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    dp, ds, dz, dx = _to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), _to_dev(x, cuda)
    dq = torch.empty((M, K), dtype=torch.float16, device=cuda)
    assert ref.ref_dequant(_ptr(dp), _ptr(ds), _ptr(dz), _ptr(dq), M, K, None) == 0
    y = torch.empty(M, dtype=torch.float16, device=cuda)
    assert ref.ref_gemv_cublas(_ptr(dq), _ptr(dx), _ptr(y), M, K, 1, None) == 0
    torch.cuda.synchronize()
    got_ref32 = y.cpu().numpy()
    # the library sums in fp32 in its own (tensor-core) order: never more than the last fp16 bit from the oracle's
    # correctly rounded sum, and that on a few percent of the outputs (measured: 1.6 %)
    for name, other in (("oracle", y16), ("product", _run_gemv(ops, cuda, p, s, z, M, K, x))):
        ulps = _ulp_diff(got_ref32, other)
        tiny = np.abs(got_ref32.astype(np.float32) - other.astype(np.float32)) <= 1e-4 * np.abs(y32).mean()
        assert ((ulps <= 1) | tiny).all(), f"{name}: {int(ulps[~tiny].max())} ulp from cuBLAS on the reference's buffer"
        assert (ulps > 0).mean() < 0.05, f"{name}: {(ulps > 0).mean():.4f} of outputs differ from cuBLAS"
    # fp16 accumulation (what the reference's fp16 alpha / beta ask for): same layout, its own rounding noise
    assert ref.ref_gemv_cublas(_ptr(dq), _ptr(dx), _ptr(y), M, K, 0, None) == 0
    torch.cuda.synchronize()
    err16 = np.abs(y.cpu().numpy().astype(np.float32) - y32)
    rms = float(np.sqrt((y32 ** 2).mean()))
    assert err16.max() <= 0.25 * rms, (float(err16.max()), rms)
