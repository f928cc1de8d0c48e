"""GPU parity of the dequantisation hook and the fused dequant-GEMV against the CPU oracle.

Bar: dequantised weights bit-exact; GEMV outputs within rtol 2e-2 of the oracle's fp32 sums (the
tolerance the task states for logits) -- in practice the fp16 results are compared much tighter:
at most a small fraction may differ, and then by one fp16 ulp (fp32 summation order only).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL = 2e-2

# (out_dim, in_dim, kind): the six matrix kinds of the model at reduced and at full size.
SHAPES_SMALL = [
    (1536, 512, "wqkv-like: out = 3*in, group independent of j"),
    (512, 512, "wo-like"),
    (512, 1536, "w2-like: reference indexes past its scale array; wrapped"),
    (1152, 512, "unembed-like: out/128 = 9 not a multiple of in/128 = 4, group depends on j"),
    (2176, 512, "unembed-like with a ragged last tile (2176 = 2*1024 + 128)"),
    (640, 384, "odd block counts"),
    (128, 128, "smallest"),
    (4096, 128, "one unit of rows"),
]
SHAPES_FULL = [(12288, 4096), (4096, 4096), (4096, 12288), (151936, 4096)]


def _to_dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _ulp_diff(a, b):
    """Distance in fp16 ulps between two float16 arrays (sign-magnitude ordered)."""
    def key(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u)
    return np.abs(key(a) - key(b))


@pytest.mark.parametrize("M,K,why", SHAPES_SMALL)
def test_dequant_bit_exact_small(ops, orc, cuda, M, K, why):
    p, s, z = orc.gen_linear(1, M, K)
    want = orc.dequant(p, s, z, M, K)
    got = ops.dequant_w4(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), M, K).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), why


def test_dequant_bit_exact_word_embedding_layout(ops, orc, cuda):
    """word_embedding is [hidden][vocab]: in_dim/128 groups are needed, hidden/128 exist (wrapped)."""
    H, V = 256, 4096 + 384
    p, s, z = orc.gen_linear(2, H, V, kind=orc.EMB)
    want = orc.dequant(p, s, z, H, V)
    got = ops.dequant_w4(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), H, V).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_dequant_bit_exact_fractional_zero_points(ops, orc, cuda):
    M, K = 512, 512
    p, s, _ = orc.gen_linear(3, M, K)
    z = (orc.gen_normal_f16(3, 999, M // 128, 7.5, 1.3)).astype(np.float16)
    want = orc.dequant(p, s, z, M, K)
    got = ops.dequant_w4(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), M, K).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def _run_gemv(ops, cuda, p, s, z, M, K, x, zp_integral=True, pdl=False, canary=True):
    ws = ops.Workspace(pdl=pdl)
    w = ops.W4Linear(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), M, K, zp_integral=zp_integral)
    pad = 256
    ybuf = torch.full((M + 2 * pad,), -7.0, dtype=torch.float16, device=cuda)
    y = ybuf[pad:pad + M]
    ops.gemv_w4a16(w, ws, ops.gemv_args(_to_dev(x, cuda), y=y))
    ws.check()
    out = ybuf.cpu().numpy()
    if canary:  # nothing outside [0, M) may be written
        assert (out[:pad] == np.float16(-7.0)).all() and (out[pad + M:] == np.float16(-7.0)).all()
    return out[pad:pad + M]


def _check_against_oracle(got, y32, y16, what):
    err = np.abs(got.astype(np.float32) - y32)
    tol = RTOL * np.abs(y32) + RTOL * np.abs(y32).mean()
    assert (err <= tol).all(), f"{what}: max err {err.max()} vs oracle"
    # fp16 results: equal, or one ulp apart where the fp32 sum sits on a rounding boundary; outputs
    # that cancel to almost nothing are compared on absolute error (an ulp there is far below the
    # fp32 summation noise of the terms that cancelled).
    ulps = _ulp_diff(got, y16)
    tiny = np.abs(got.astype(np.float32) - y16.astype(np.float32)) <= 1e-4 * np.abs(y32).mean()
    assert ((ulps <= 1) | tiny).all(), f"{what}: {ulps[~tiny].max()} ulp from the oracle's fp16 result"
    assert (ulps > 0).mean() < 0.01, f"{what}: {(ulps > 0).mean():.4f} of outputs differ from the oracle"


@pytest.mark.parametrize("M,K,why", SHAPES_SMALL)
def test_gemv_matches_oracle_small(ops, orc, cuda, M, K, why):
    p, s, z = orc.gen_linear(0, M, K)
    x = orc.gen_normal_f16(0, orc.ACT, K)
    y32, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    got = _run_gemv(ops, cuda, p, s, z, M, K, x)
    _check_against_oracle(got, y32, y16, why)


@pytest.mark.parametrize("M,K", [(512, 512), (1152, 512)])
def test_gemv_fractional_zero_points(ops, orc, cuda, M, K):
    p, s, _ = orc.gen_linear(5, M, K)
    z = orc.gen_normal_f16(5, 999, M // 128, 7.5, 1.3)
    x = orc.gen_normal_f16(5, orc.ACT, K)
    y32, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    got = _run_gemv(ops, cuda, p, s, z, M, K, x, zp_integral=False)
    _check_against_oracle(got, y32, y16, "generic zero-point path")


def test_gemv_single_awq_linear_seed0(ops, orc, cuda):
    """The single-linear configuration: N=4096 x K=4096, seed 0, x ~ N(0,1)."""
    M = K = 4096
    p, s, z = orc.gen_linear(0, M, K)
    x = orc.gen_normal_f16(0, orc.ACT, K)
    y32, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    for pdl in (False, True):
        got = _run_gemv(ops, cuda, p, s, z, M, K, x, pdl=pdl)
        _check_against_oracle(got, y32, y16, f"4096x4096 pdl={pdl}")


@pytest.mark.parametrize("M,K", SHAPES_FULL)
def test_gemv_full_size_shapes(ops, orc, cuda, M, K):
    kind = orc.UNEMB if M == 151936 else orc.WQKV
    p, s, z = orc.gen_linear(0, M, K, kind=kind)
    x = orc.gen_normal_f16(0, orc.ACT, K)
    y32, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    got = _run_gemv(ops, cuda, p, s, z, M, K, x)
    _check_against_oracle(got, y32, y16, f"{M}x{K}")


def test_gemv_is_deterministic_and_linear(ops, orc, cuda):
    """Size-independent properties at a full-size shape: bitwise repeatable; y(2x) = 2 y(x) exactly
    (scaling by two is exact in fp16 and fp32)."""
    M, K = 12288, 4096
    p, s, z = orc.gen_linear(7, M, K)
    x = orc.gen_normal_f16(7, orc.ACT, K)
    a = _run_gemv(ops, cuda, p, s, z, M, K, x)
    b = _run_gemv(ops, cuda, p, s, z, M, K, x)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    c = _run_gemv(ops, cuda, p, s, z, M, K, (x.astype(np.float32) * 2).astype(np.float16))
    assert np.array_equal((a.astype(np.float32) * 2).astype(np.float16).view(np.uint16), c.view(np.uint16))


def test_gemv_epilogues(ops, orc, cuda):
    M, K = 1536, 512
    p, s, z = orc.gen_linear(9, M, K)
    x = orc.gen_normal_f16(9, orc.ACT, K)
    gamma = orc.gen_normal_f16(9, orc.GAMMA, K, 1.0, 0.02)
    ws = ops.Workspace()
    w = ops.W4Linear(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), M, K)
    xd, gd = _to_dev(x, cuda), _to_dev(gamma, cuda)
    # RMSNorm prologue + GeLU epilogue
    xn = orc.rmsnorm(x, gamma)
    _, y16 = orc.gemm_w4a16(p, s, z, M, K, xn)
    want = orc.gelu(y16)
    y = torch.zeros(M, dtype=torch.float16, device=cuda)
    ops.gemv_w4a16(w, ws, ops.gemv_args(xd, epilogue=ops.cabi.EPI_GELU, y=y, gamma=gd))
    got = y.cpu().numpy()
    # a one-ulp difference of the GEMV result may move the GeLU output by a few ulps where GeLU is
    # steep relative to its value (negative tail); compare those on absolute error
    d = _ulp_diff(got, want)
    near = np.abs(got.astype(np.float32) - want.astype(np.float32)) <= 1e-3 * np.abs(want.astype(np.float32)).mean()
    assert ((d <= 2) | near).all() and (d > 0).mean() < 0.02
    # residual epilogue, no prologue
    res = orc.gen_normal_f16(10, orc.ACT, M)
    _, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    want = orc.add(res, y16)
    y = _to_dev(res, cuda).clone()
    ops.gemv_w4a16(w, ws, ops.gemv_args(xd, epilogue=ops.cabi.EPI_RESIDUAL, y=y))
    got = y.cpu().numpy()
    assert _ulp_diff(got, want).max() <= 1 and (_ulp_diff(got, want) > 0).mean() < 0.01
    ws.check()


def test_gemv_rope_kv_epilogue(ops, orc, cuda):
    heads, max_pos, pos = 4, 64, 37
    H = heads * 128
    M, K = 3 * H, H
    p, s, z = orc.gen_linear(11, M, K)
    x = orc.gen_normal_f16(11, orc.ACT, K)
    cos_t, sin_t = orc.rope_tables(max_pos, 128, 1e6)
    _, qkv = orc.gemm_w4a16(p, s, z, M, K, x)
    q_want = orc.rope(qkv[:H], heads, 128, cos_t, sin_t, pos)
    k_want = orc.rope(qkv[H:2 * H], heads, 128, cos_t, sin_t, pos)
    v_want = qkv[2 * H:]
    ws = ops.Workspace()
    w = ops.W4Linear(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), M, K)
    q = torch.zeros(H, dtype=torch.float16, device=cuda)
    kc = torch.zeros(heads, max_pos, 128, dtype=torch.float16, device=cuda)
    vc = torch.zeros_like(kc)
    d_pos = torch.tensor([pos], dtype=torch.int32, device=cuda)
    ops.gemv_w4a16(w, ws, ops.gemv_args(_to_dev(x, cuda), epilogue=ops.cabi.EPI_ROPE_KV, y=q, k_cache=kc, v_cache=vc,
                                        cos=_to_dev(cos_t, cuda), sin=_to_dev(sin_t, cuda), heads=heads, max_pos=max_pos,
                                        d_pos=d_pos))
    ws.check()
    for got, want in ((q.cpu().numpy(), q_want), (kc[:, pos].reshape(-1).cpu().numpy(), k_want),
                      (vc[:, pos].reshape(-1).cpu().numpy(), v_want)):
        d = _ulp_diff(got, want)
        assert d.max() <= 4 and (d > 0).mean() < 0.02   # a 1-ulp GEMV difference passes through 3 fp16 ops
    kc[:, pos] = 0
    vc[:, pos] = 0
    assert not kc.any() and not vc.any()    # no other cache row was touched


def test_gemv_argmax_epilogue(ops, orc, cuda):
    M, K = 2176, 512
    p, s, z = orc.gen_linear(13, M, K, kind=orc.UNEMB)
    x = orc.gen_normal_f16(13, orc.ACT, K)
    _, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    ws = ops.Workspace()
    w = ops.W4Linear(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), M, K)
    logits = torch.zeros(M, dtype=torch.float16, device=cuda)
    l32 = torch.zeros(M, dtype=torch.float32, device=cuda)
    tok = torch.full((1,), -1, dtype=torch.int32, device=cuda)
    for _ in range(2):   # twice: the arrival counters must reset themselves
        ops.gemv_w4a16(w, ws, ops.gemv_args(_to_dev(x, cuda), epilogue=ops.cabi.EPI_ARGMAX, y=logits, d_token=tok, logits_f32=l32))
    ws.check()
    got = logits.cpu().numpy()
    assert _ulp_diff(got, y16).max() <= 1
    assert int(tok.item()) == orc.argmax_f16(got)
    assert np.array_equal(l32.cpu().numpy(), got.astype(np.float32))


def test_bad_arguments_are_rejected(ops, orc, cuda):
    import ctypes as C
    cabi = ops.cabi
    p, s, z = orc.gen_linear(0, 256, 128)
    with pytest.raises(cabi.Qw3Error) as e:
        ops.W4Linear(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), 200, 128)
    assert e.value.status == cabi.QW3_ERR_ARG
    w = ops.W4Linear(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), 256, 128)
    ws = ops.Workspace()
    with pytest.raises(cabi.Qw3Error):
        ops.gemv_w4a16(w, ws, ops.gemv_args(None, y=torch.zeros(256, dtype=torch.float16, device=cuda)))
