"""Host logic of the fused token pass: the work split (qw3_fused_plan) and the load-time repack of the on-disk
nibble stream into per-(CTA, warp) streams (qw3_fused_repack_host), checked by replaying on the CPU exactly what a
warp of fused_pass_kernel does with its stream -- 16-byte pieces per lane, the four masks that turn a word into the
m16n8k16 A fragment, the B fragment taken from the activations in stream order -- and comparing the sums with the
contraction the reference defines (Inference.cu:1052-1065 over the flat nibble stream of Inference.cu:84-105)."""
import ctypes as C

import numpy as np
import pytest

SMALL = dict(hidden=512, inter=1536, heads=4, head_dim=128, layers=4, vocab=2176, max_pos=64)
QKV, WO, W1, W2, UNEMB = range(5)


def _plan(pkg, cfg_kw, n_ranks=1, rank=0, grid=148):
    cabi = pkg.cabi
    cfg = cabi.default_config(**cfg_kw)
    geom = (C.c_int32 * 16)()
    plans = (C.c_int32 * 50)()
    cabi.check(cabi.lib().qw3_fused_plan(C.byref(cfg), n_ranks, rank, grid, geom, plans), "qw3_fused_plan")
    names = ["H", "I", "heads", "vocab", "n_ranks", "rank", "heads_local", "gs", "n_act", "rs", "n1", "n_blocks", "grid", "n_mlp"]
    g = dict(zip(names, list(geom)))
    pn = ["n_cta", "n_mt", "n_ks", "wk", "tb", "nb", "nq", "rem", "warp_bytes", "unit_bytes"]
    return cfg, g, [dict(zip(pn, list(plans)[10 * k:10 * k + 10])) for k in range(5)]


def test_plan_of_the_full_model(pkg):
    _, g, pl = _plan(pkg, dict(max_pos=40960))
    assert (g["gs"], g["n_act"], g["rs"], g["n1"], g["n_blocks"]) == (4, 128, 32, 96, 1187)
    # per layer every CTA that runs the layers streams 1/128 of the four matrices, every warp 1/16 of that
    per_warp = sum(pl[k]["warp_bytes"] for k in (QKV, WO, W1, W2))
    assert per_warp * 16 * 128 == 25165824 + 8388608 + 25165824 + 25165824
    assert pl[UNEMB]["warp_bytes"] * 16 == 128 * 4096 // 2
    for p in pl:
        assert p["n_mt"] == (16 // p["wk"]) * p["nb"] * p["tb"] and p["n_ks"] == p["wk"] * (4 * p["nq"] + p["rem"])
        assert p["rem"] in (0, 2) and (p["rem"] == 0 or p["tb"] % 2 == 0)
        group = p["tb"] * 512
        assert p["unit_bytes"] == (p["tb"] * (p["nq"] * 512 + p["rem"] * 128) if p["rem"] else p["unit_bytes"] // group * group)


def test_plan_of_the_full_model_in_clusters(pkg):
    """With the head groups as thread-block clusters of four CTAs only 33 clusters are co-resident on the part: the grid
    is 132 CTAs.  Same work split for the layers; the 1187 blocks of the unembedding then take nine full rounds."""
    _, g148, pl148 = _plan(pkg, dict(max_pos=40960))
    _, g, pl = _plan(pkg, dict(max_pos=40960), grid=132)
    assert (g["gs"], g["n_act"], g["rs"], g["n1"], g["grid"]) == (4, 128, 32, 96, 132)
    assert pl[:4] == pl148[:4]
    assert -(-g["n_blocks"] // 132) == 9 and 9 * 132 - g["n_blocks"] == 1


@pytest.mark.parametrize("n_ranks", [2, 4, 8])
def test_plan_of_the_full_model_row_split(pkg, n_ranks):
    """Every matrix row-split over 2, 4 and 8 GPUs: all 128 CTAs of a GPU share its heads, the bytes divide by the GPUs."""
    _, g, pl = _plan(pkg, dict(max_pos=40960), n_ranks, n_ranks - 1)
    assert g["n_act"] == 128 and g["gs"] == 4 * n_ranks and g["rs"] == 32 // n_ranks
    assert g["n_mlp"] * g["n1"] * n_ranks == 12288 and g["n1"] % 32 == 0
    per_gpu = 16 * (128 * (pl[QKV]["warp_bytes"] + pl[WO]["warp_bytes"]) + g["n_mlp"] * (pl[W1]["warp_bytes"] + pl[W2]["warp_bytes"]))
    assert per_gpu * n_ranks == 25165824 + 8388608 + 25165824 + 25165824


def test_unsupported_shapes_are_refused(pkg):
    cabi = pkg.cabi
    cfg = cabi.default_config(hidden=384, heads=3, inter=1536, vocab=2176, layers=2, max_pos=64)   # an odd head count
    geom = (C.c_int32 * 16)()
    plans = (C.c_int32 * 50)()
    rc = cabi.lib().qw3_fused_plan(C.byref(cfg), 1, 0, 148, geom, plans)
    assert rc in (cabi.QW3_OK, cabi.QW3_ERR_ARG)   # either covered or refused with a status, never a crash
    cfg = cabi.default_config(hidden=8192, heads=64, inter=12288, vocab=2176, layers=2, max_pos=64)
    assert cabi.lib().qw3_fused_plan(C.byref(cfg), 1, 0, 148, geom, plans) == cabi.QW3_ERR_ARG     # hidden beyond the kernel's buffers


def _tile_out(g, op, cta, tile, blk):
    if op == QKV:
        head = g["rank"] * g["heads_local"] + cta // g["gs"]
        return (tile // 8) * g["H"] + head * 128 + (tile % 8) * 16
    if op == WO:
        return (cta % g["gs"]) * (g["H"] // g["gs"]) + tile * 16
    if op == W1:
        return (g["rank"] * g["n_mlp"] + cta) * g["n1"] + tile * 16
    if op == W2:
        return tile * 16
    return blk * 128 + tile * 16


def _k0(g, op, cta):
    if op == QKV:
        return (cta % g["gs"]) * (g["H"] // g["gs"])
    if op == WO:
        return (g["rank"] * g["heads_local"] + cta // g["gs"]) * 128
    if op == W2:
        return (g["rank"] * g["n_mlp"] + cta) * g["n1"]
    return 0


def _warp_streams(stream_words, p):
    """The ring's view of a CTA's stream: unit after unit, a unit being [warp][piece of unit_bytes] (whole k-groups);
    returns the 16 per-warp streams."""
    wb, ub, out, at = p["warp_bytes"], p["unit_bytes"], [[] for _ in range(16)], 0
    assert wb % ub == 0 and ub <= 4096 and ub % 256 == 0
    for _ in range(wb // ub):
        for warp in range(16):
            out[warp].append(stream_words[at:at + ub // 4])
            at += ub // 4
    assert at == stream_words.size
    return np.concatenate([np.concatenate(w) for w in out])


def _consume(stream_words, p, g, op, cta, blk, x, y):
    """What the 16 warps of one CTA do with their streams (gemv_core of fused_pass.cu), in integers."""
    stream_words = _warp_streams(stream_words, p)
    ksw = 4 * p["nq"] + p["rem"]
    x_cta = x[_k0(g, op, cta):]
    lanes = np.arange(32)
    gq, t = lanes >> 2, lanes & 3
    wpw = p["warp_bytes"] // 4
    for warp in range(16):
        a, bk = warp // p["wk"], warp % p["wk"]
        xs = x_cta[bk * ksw * 16:]
        words = stream_words[warp * wpw:(warp + 1) * wpw]
        off = 0
        for b in range(p["nb"]):
            acc = np.zeros((p["tb"], 16), np.int64)
            groups = [(q, 4) for q in range(p["nq"])] + ([(p["nq"], 2)] if p["rem"] == 2 else [])
            for q, steps in groups:
                for i in range(p["tb"]):
                    item = words[off:off + 32 * steps].reshape(32, steps)   # lane-major: `steps` words per lane
                    off += 32 * steps
                    for s in range(steps):
                        w = item[:, s].astype(np.int64)
                        xb = q * 64 + 4 * steps * t + 4 * s                # B fragment: byte k of this lane's register s = x[xb + k]
                        lo = sum(((w >> (8 * k)) & 0xF) * xs[xb + k] for k in range(4))        # w & 0x0f0f0f0f: rows g
                        hi = sum(((w >> (8 * k + 4)) & 0xF) * xs[xb + k] for k in range(4))    # w & 0xf0f0f0f0: rows g + 8 (x 16 in the MMA)
                        np.add.at(acc[i], gq, lo)
                        np.add.at(acc[i], gq + 8, hi)
            for i in range(p["tb"]):
                tile = a * (p["nb"] * p["tb"]) + b * p["tb"] + i
                o = _tile_out(g, op, cta, tile, blk)
                y[o:o + 16] += acc[i]
        assert off == wpw


@pytest.mark.parametrize("n_ranks,rank,grid", [(1, 0, 24), (1, 0, 8), (2, 1, 8)])
@pytest.mark.parametrize("op", [QKV, WO, W1, W2, UNEMB])
def test_repacked_streams_reproduce_the_contraction(pkg, op, n_ranks, rank, grid):
    cabi = pkg.cabi
    try:
        cfg, g, pl = _plan(pkg, SMALL, n_ranks, rank, grid)
    except cabi.Qw3Error:
        pytest.skip("this split is not covered by the fused pass")
    p = pl[op]
    H, I, V = SMALL["hidden"], SMALL["inter"], SMALL["vocab"]
    M, K = {QKV: (3 * H, H), WO: (H, H), W1: (I, H), W2: (H, I), UNEMB: (V, H)}[op]
    rng = np.random.default_rng(op * 7 + rank)
    raw = rng.integers(0, 256, M * K // 2, dtype=np.uint8)
    x = rng.integers(-8, 9, K).astype(np.int64)
    n_rounds = -(-g["n_blocks"] // (n_ranks * grid))
    streams = n_rounds * grid if op == UNEMB else p["n_cta"]
    out = np.zeros(streams * 16 * p["warp_bytes"], np.uint8)
    cabi.check(cabi.lib().qw3_fused_repack_host(C.byref(cfg), n_ranks, rank, grid, op, raw.ctypes.data_as(C.c_void_p), M,
                                                out.ctypes.data_as(C.c_void_p), out.size), "qw3_fused_repack_host")
    words = out.view(np.uint32)
    wps = 16 * p["warp_bytes"] // 4
    y = np.zeros(M, np.int64)
    covered = np.zeros(M, bool)
    for st in range(streams):
        cta = st % grid if op == UNEMB else st
        blk = ((st // grid) * n_ranks + rank) * grid + cta if op == UNEMB else 0
        if op == UNEMB and blk >= g["n_blocks"]:
            assert not words[st * wps:(st + 1) * wps].any()
            continue
        _consume(words[st * wps:(st + 1) * wps], p, g, op, cta, blk, x, y)
        for tile in range(p["n_mt"]):
            o = _tile_out(g, op, cta, tile, blk)
            covered[o:o + 16] = True
    # the reference's contraction on the same bytes: y[i] = sum_j q(i + j*M) x[j], restricted to what this rank holds
    nib = np.empty(M * K, np.int64)
    nib[0::2] = raw & 15
    nib[1::2] = raw >> 4
    q = nib.reshape(K, M)            # q[j, i] = flat element i + j*M
    if op in (QKV, WO, W2):
        # inputs are split: this rank multiplies only its heads' / its W1 outputs' columns
        kmask = np.zeros(K, bool)
        for cta in range(p["n_cta"]):
            k0 = _k0(g, op, cta)
            kmask[k0:k0 + p["n_ks"] * 16] = True
        want = (q[kmask].T * x[kmask]).sum(axis=1)
    else:
        want = (q.T * x).sum(axis=1)
    assert covered.any()
    assert (y[covered] == want[covered]).all()
    if n_ranks == 1:
        assert covered.all()
