"""GPU parity of the small operators (RMSNorm, RoPE + KV append, decode attention, embedding
gather, arg-max) against the CPU oracle."""
import numpy as np
import pytest
import torch

from test_gemv_gpu import _to_dev, _ulp_diff

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [128, 512, 4096, 12288])
def test_rmsnorm_bit_exact(ops, orc, cuda, n):
    x = orc.gen_normal_f16(21, orc.ACT, n, 0.0, 3.0)
    g = orc.gen_normal_f16(21, orc.GAMMA, n, 1.0, 0.02)
    want = orc.rmsnorm(x, g)
    got = ops.rmsnorm(_to_dev(x, cuda), _to_dev(g, cuda)).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def test_rope_kv_append_bit_exact(ops, orc, cuda):
    heads, max_pos = 8, 128
    H = heads * 128
    qkv = orc.gen_normal_f16(22, orc.ACT, 3 * H)
    cos_t, sin_t = orc.rope_tables(max_pos, 128, 10000.0)
    for pos in (0, 1, 77, 127):
        q = torch.zeros(H, dtype=torch.float16, device=cuda)
        kc = torch.zeros(heads, max_pos, 128, dtype=torch.float16, device=cuda)
        vc = torch.zeros_like(kc)
        ops.rope_kv_append(_to_dev(qkv, cuda), q, kc, vc, _to_dev(cos_t, cuda), _to_dev(sin_t, cuda), heads, max_pos, pos)
        assert np.array_equal(q.cpu().numpy().view(np.uint16), orc.rope(qkv[:H], heads, 128, cos_t, sin_t, pos).view(np.uint16))
        assert np.array_equal(kc[:, pos].reshape(-1).cpu().numpy().view(np.uint16),
                              orc.rope(qkv[H:2 * H], heads, 128, cos_t, sin_t, pos).view(np.uint16))
        assert np.array_equal(vc[:, pos].reshape(-1).cpu().numpy().view(np.uint16), qkv[2 * H:].view(np.uint16))


@pytest.mark.parametrize("heads,max_pos,length", [(4, 64, 1), (4, 64, 2), (8, 600, 513), (32, 1024, 512), (32, 2048, 2048), (2, 4096, 3000)])
def test_attention_decode(ops, orc, cuda, heads, max_pos, length):
    q = orc.gen_normal_f16(23, orc.ACT, heads * 128)
    kc = orc.gen_normal_f16(23, orc.KV_K, heads * max_pos * 128)
    vc = orc.gen_normal_f16(23, orc.KV_V, heads * max_pos * 128)
    want = orc.attention(q, kc, vc, heads, 128, max_pos, length)
    ws = ops.Workspace()
    for _ in range(2):
        got = ops.attn_decode(_to_dev(q, cuda), _to_dev(kc, cuda), _to_dev(vc, cuda), heads, max_pos, length - 1, ws).cpu().numpy()
    ws.check()
    err = np.abs(got.astype(np.float32) - want.astype(np.float32))
    assert (err <= 2e-2 * np.abs(want.astype(np.float32)) + 2e-3).all()
    d = _ulp_diff(got, want)
    assert (d > 1).mean() < 0.01


@pytest.mark.parametrize("heads,max_pos,pos0,rows", [(4, 256, 0, 64), (4, 600, 100, 37), (32, 1024, 256, 256), (2, 4096, 3000, 130),
                                                     (4, 64, 3, 5), (3, 300, 0, 16), (2, 700, 511, 129)])
def test_attention_prefill_block(ops, orc, cuda, heads, max_pos, pos0, rows):
    """A block of prompt rows: row r must equal the oracle's attention of its q over cache rows 0 .. pos0 + r.  Blocks
    that start inside a tile, end inside a row block, sit far from position 0, and blocks of a few rows (one CTA per row)."""
    H = heads * 128
    qkv = orc.gen_normal_f16(29, orc.ACT, rows * 3 * H).reshape(rows, 3 * H)
    kc = orc.gen_normal_f16(29, orc.KV_K, heads * max_pos * 128)
    vc = orc.gen_normal_f16(29, orc.KV_V, heads * max_pos * 128)
    got = ops.attn_prefill(_to_dev(qkv, cuda), _to_dev(kc, cuda), _to_dev(vc, cuda), heads, max_pos, pos0, rows).cpu().numpy()
    check = sorted(set([0, 1, 15, 16, 63, 64, rows // 2, rows - 2, rows - 1]) & set(range(rows)))
    for r in check:
        want = orc.attention(np.ascontiguousarray(qkv[r, :H]), kc, vc, heads, 128, max_pos, pos0 + r + 1)
        err = np.abs(got[r].astype(np.float32) - want.astype(np.float32))
        assert (err <= 2e-2 * np.abs(want.astype(np.float32)) + 2e-3).all(), r
        assert (_ulp_diff(got[r], want) > 1).mean() < 0.01, r


def test_embed_gather_bit_exact(ops, orc, cuda):
    H, V = 512, 4096 + 256
    p, s, z = orc.gen_linear(24, H, V, kind=orc.EMB)
    pd, sd, zd = _to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda)
    for tok in (0, 1, 127, 128, 4095, 4096, V - 1):
        want = orc.embed_gather(p, s, z, H, V, tok)
        got = ops.embed_gather_w4(pd, sd, zd, H, V, tok).cpu().numpy()
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), tok
    d_tok = torch.tensor([777], dtype=torch.int32, device=cuda)
    got = ops.embed_gather_w4(pd, sd, zd, H, V, 0, d_token=d_tok).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), orc.embed_gather(p, s, z, H, V, 777).view(np.uint16))


def test_argmax_first_max_wins(ops, orc, cuda):
    n = 151936
    logits = orc.gen_normal_f16(25, orc.ACT, n)
    ws = ops.Workspace()
    assert int(ops.argmax_f16(_to_dev(logits, cuda), ws).item()) == orc.argmax_f16(logits)
    logits[:] = np.float16(1.5)   # all equal: index 0
    assert int(ops.argmax_f16(_to_dev(logits, cuda), ws).item()) == 0
    logits[100000] = np.float16(2.0)
    logits[140000] = np.float16(2.0)   # tie between two maxima: the lower index
    assert int(ops.argmax_f16(_to_dev(logits, cuda), ws).item()) == 100000
    ws.check()


def test_a_device_wait_that_runs_out_is_reported_and_leaves_the_gpu_usable(ops, orc, cuda):
    """The hand-off protocol's wait kernel on a flag nobody sets, with a limit of about two milliseconds: the kernel
    returns by itself, the workspace reports QW3_ERR_TIMEOUT with the code it was given, and the same workspace then
    runs a GEMV correctly.  Nothing faults or hangs: the wait is bounded by design and this is its limit being reached."""
    import ctypes as C
    cabi = ops.cabi
    ws = ops.Workspace()
    flag = torch.zeros(4, dtype=torch.int32, device=cuda)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    cabi.check(cabi.lib().qw3_handoff_wait(C.c_void_p(flag.data_ptr()), 1, 4_000_000, 0x40005, ws.h, st), "qw3_handoff_wait")
    with pytest.raises(cabi.Qw3Error) as e:
        ws.check()
    assert e.value.status == cabi.QW3_ERR_TIMEOUT and b"0x40005" in cabi.lib().qw3_last_error()
    ws.check()   # the word was cleared by the failing check
    # a flag that is already set: the same launch returns without an error
    flag[0] = 3
    cabi.check(cabi.lib().qw3_handoff_wait(C.c_void_p(flag.data_ptr()), 2, 4_000_000, 0x40005, ws.h, st), "qw3_handoff_wait")
    ws.check()
    M, K = 1536, 512
    p, s, z = orc.gen_linear(41, M, K)
    x = orc.gen_normal_f16(41, orc.ACT, K)
    w = ops.W4Linear(_to_dev(p, cuda), _to_dev(s, cuda), _to_dev(z, cuda), M, K)
    y = torch.zeros(M, dtype=torch.float16, device=cuda)
    ops.gemv_w4a16(w, ws, ops.gemv_args(_to_dev(x, cuda), y=y))
    ws.check()
    y32, _ = orc.gemm_w4a16(p, s, z, M, K, x)
    err = np.abs(y.cpu().numpy().astype(np.float32) - y32)
    assert (err <= 2e-2 * np.abs(y32) + 2e-2 * np.abs(y32).mean()).all()
