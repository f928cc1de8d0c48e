"""CPU checks of the oracle: against an independent numpy restatement, against the committed
golden fixtures, and for the properties the kernels rely on (group formula, determinism)."""
import json
import os

import numpy as np
import pytest

import np_ref

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "golden.json")))


def bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def test_generator_matches_numpy_restatement(orc):
    for seed, tag, n in [(0, 0, 1003), (7, 12345, 64), (2**40 + 3, 9, 17)]:
        assert np.array_equal(orc.gen_codes(seed, tag, n), np_ref.gen_codes(seed, tag, n))
        assert np.array_equal(orc.gen_uniform_int_f16(seed, tag, n, 6, 9), np_ref.gen_uniform_int_f16(seed, tag, n, 6, 9))
        assert np.array_equal(orc.gen_tokens(seed, tag, n, 151936), np_ref.gen_tokens(seed, tag, n, 151936))
        a = orc.gen_normal_f16(seed, tag, n).astype(np.float32)
        b = np_ref.gen_normal(seed, tag, n).astype(np.float16).astype(np.float32)
        assert (a == b).mean() > 0.999   # libm vs numpy log/cos may differ in the last place


def test_generator_distributions(orc):
    p, s, z = orc.gen_linear(0, 4096, 4096)
    lo, hi = p & 15, p >> 4
    counts = np.bincount(np.concatenate([lo[:1 << 20], hi[:1 << 20]]), minlength=16) / (1 << 21)
    assert np.abs(counts - 1 / 16).max() < 2e-3                      # codes uniform 0..15
    assert set(np.unique(z.astype(np.float32))) <= {6.0, 7.0, 8.0, 9.0}
    big = orc.gen_normal_f16(0, 1, 1 << 16, 0.0, 0.02, True).astype(np.float32)
    assert (big >= 0).all() and abs(big.mean() - 0.02 * np.sqrt(2 / np.pi)) < 3e-4
    x = orc.gen_normal_f16(0, orc.ACT, 1 << 16).astype(np.float32)
    assert abs(x.mean()) < 0.02 and abs(x.std() - 1) < 0.02


def test_generator_golden(orc):
    g = GOLDEN["generator"]
    assert orc.gen_codes(0, 0, 32).tobytes().hex() == g["codes_seed0_tag0"]
    assert orc.gen_normal_f16(0, 1, 8, 0.0, 0.02, True).tobytes().hex() == g["scale_seed0_tag1"]
    assert orc.gen_uniform_int_f16(0, 2, 8, 6, 9).tobytes().hex() == g["zp_seed0_tag2"]
    assert orc.gen_normal_f16(0, orc.ACT, 8).tobytes().hex() == g["act_seed0"]
    assert [int(t) for t in orc.gen_tokens(0, orc.TOKENS, 8, 151936)] == g["tokens_seed0"]


SHAPES = [(256, 128), (384, 128), (128, 384), (1152, 512), (512, 1536), (640, 384), (2176, 512)]


@pytest.mark.parametrize("M,K", SHAPES)
def test_dequant_bit_exact_two_implementations(orc, M, K):
    p, s, z = orc.gen_linear(3, M, K)
    assert np.array_equal(bits(orc.dequant(p, s, z, M, K)), bits(np_ref.dequant(p, s, z, M, K)))
    zf = orc.gen_normal_f16(3, 999, M // 128, 7.5, 1.3)    # fractional zero-points round in the subtraction
    assert np.array_equal(bits(orc.dequant(p, s, zf, M, K)), bits(np_ref.dequant(p, s, zf, M, K)))


def test_dequant_wraps_group_index_past_the_allocation(orc):
    """word_embedding-like [hidden][vocab]: vocab/128 groups are indexed, hidden/128 exist."""
    H, V = 256, 1280
    p, s, z = orc.gen_linear(4, H, V, kind=orc.EMB)
    d = orc.dequant(p, s, z, H, V)
    assert np.array_equal(bits(d), bits(np_ref.dequant(p, s, z, H, V)))
    q = np_ref.unpack_nibbles(p, H, V)
    c = 5 * 128 + 3                                           # group 5 -> entry 5 mod 2 = 1
    want = ((q[:, c].astype(np.float16) - z[1]) * s[1]).astype(np.float16)
    assert np.array_equal(bits(d[:, c]), bits(want))


@pytest.mark.parametrize("M,K", SHAPES)
def test_gemv_matches_float64_and_scalar_path(orc, M, K):
    p, s, z = orc.gen_linear(0, M, K)
    x = orc.gen_normal_f16(0, orc.ACT, K)
    y32, y16 = orc.gemm_w4a16(p, s, z, M, K, x)               # AVX2, double accumulation
    ys32, _ = orc.gemm_w4a16(p, s, z, M, K, x, acc64=False)   # scalar, float accumulation
    yn = np_ref.gemv(p, s, z, M, K, x)                        # numpy float64 on the numpy dequant
    scale = np.abs(yn).max()
    assert np.abs(y32 - yn).max() <= 1e-6 * scale
    assert np.abs(ys32 - yn).max() <= 1e-5 * scale
    assert np.array_equal(bits(y16), bits(y32.astype(np.float16)))


@pytest.mark.parametrize("M,K", SHAPES + [(12288, 4096), (4096, 12288), (151936, 4096)])
def test_group_closed_form_equals_flat_index_rule(M, K):
    n_alloc = M // 128
    if M * K > 1 << 24:   # sample rows of the big shapes
        i = np.arange(0, M, 97, dtype=np.int64)[:, None]
        j = np.arange(K, dtype=np.int64)[None, :]
        brute = (((i + j * M) % K) // 128) % n_alloc
        closed = (((i // 128) + j * (M // 128)) % (K // 128)) % n_alloc
        assert np.array_equal(brute, closed)
    else:
        assert np.array_equal(np_ref.group_index_bruteforce(M, K, 128, n_alloc), np_ref.group_index_blocked(M, K, 128, n_alloc))


def test_gemm_rows_equal_gemv(orc):
    M, K, R = 384, 256, 5
    p, s, z = orc.gen_linear(6, M, K)
    X = orc.gen_normal_f16(6, orc.ACT, R * K).reshape(R, K)
    Y32, Y16 = orc.gemm_w4a16(p, s, z, M, K, X)
    for r in range(R):
        y32, y16 = orc.gemm_w4a16(p, s, z, M, K, X[r])
        assert np.array_equal(y32, Y32[r]) and np.array_equal(bits(y16), bits(Y16[r]))


def test_small_operators_match_numpy(orc):
    n = 4096
    x = orc.gen_normal_f16(8, orc.ACT, n, 0.0, 3.0)
    g = orc.gen_normal_f16(8, orc.GAMMA, n, 1.0, 0.02)
    assert np.array_equal(bits(orc.rmsnorm(x, g)), bits(np_ref.rmsnorm(x, g).astype(np.float16)))
    heads = 4
    cos_t, sin_t = orc.rope_tables(64, 128, 10000.0)
    qk = orc.gen_normal_f16(8, orc.ACT, heads * 128)
    for pos in (0, 1, 63):
        assert np.array_equal(bits(orc.rope(qk, heads, 128, cos_t, sin_t, pos)), bits(np_ref.rope(qk, heads, 128, cos_t, sin_t, pos)))
    max_pos, length = 96, 70
    kc = orc.gen_normal_f16(8, orc.KV_K, heads * max_pos * 128)
    vc = orc.gen_normal_f16(8, orc.KV_V, heads * max_pos * 128)
    a = orc.attention(qk, kc, vc, heads, 128, max_pos, length).astype(np.float32)
    b = np_ref.attention(qk, kc, vc, heads, 128, max_pos, length)
    assert np.abs(a - b).max() <= 2e-3 * max(1.0, np.abs(b).max())
    ge = orc.gelu(x).astype(np.float32)
    assert np.abs(ge - np_ref.gelu(x)).max() <= 2e-3 * np.abs(ge).max()
    y = orc.gen_normal_f16(9, orc.ACT, n)
    assert np.array_equal(bits(orc.add(x, y)), bits(x + y))
    logits = orc.gen_normal_f16(10, orc.ACT, 5000)
    logits[4000] = logits.max()
    first = int(np.flatnonzero(logits == logits.max())[0])
    assert orc.argmax_f16(logits) == first


def test_rope_table_uses_the_configured_base(orc):
    c4, _ = orc.rope_tables(8, 128, 10000.0)
    c6, _ = orc.rope_tables(8, 128, 1e6)
    assert np.array_equal(bits(c4[:, 0]), bits(c6[:, 0])) and not np.array_equal(bits(c4), bits(c6))
    want = np.float16(np.cos(np.float32(3.0) * (np.float32(1.0) / np.float32(10000.0) ** np.float32(2 / 128))))
    assert abs(float(c4[3, 1]) - float(want)) <= 1e-3


def test_single_linear_golden(orc):
    g = GOLDEN["single_linear"]
    import hashlib
    M, K = g["M"], g["K"]
    p, s, z = orc.gen_linear(g["seed"], M, K)
    x = orc.gen_normal_f16(g["seed"], orc.ACT, K)
    assert hashlib.sha256(p.tobytes()).hexdigest() == g["packed_sha256"]
    assert hashlib.sha256(orc.dequant(p, s, z, M, K).tobytes()).hexdigest() == g["dequant_sha256"]
    y32, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    assert hashlib.sha256(y16.tobytes()).hexdigest() == g["y_f16_sha256"]
    assert y16[:8].tobytes().hex() == g["y_f16_head"]


SMALL = dict(hidden=512, inter=1536, heads=4, head_dim=128, layers=4, vocab=2176, max_pos=64, rope_base=10000.0)


def test_small_model_golden_and_weight_dir_round_trip(orc, tmp_path):
    g = GOLDEN["small_model"]
    seed = g["seed"]
    cfg = orc.default_config(**SMALL)
    prompt = orc.gen_tokens(seed, orc.TOKENS, g["n_prompt"], cfg.vocab)
    m = orc.Model(cfg)
    m.init_random(seed)
    ids, logits, margins = m.generate(prompt, g["max_new"])
    assert [int(t) for t in ids] == g["ids"]
    # the probing form of the same flow: same ids, its per-step top-8 and hidden probes are what golden.json holds
    t = m.generate_trace(prompt, g["max_new"], g["probe_layers"], g["probe_pos"])
    assert [int(v) for v in t["ids"]] == g["ids"]
    assert [[int(v) for v in r] for r in t["top_idx"]] == g["steps_top8_idx"]
    assert np.array_equal(t["top_val"].astype(np.float32), np.array(g["steps_top8"], np.float32))
    assert (t["top_idx"][:, 0] == t["ids"]).all() and (np.diff(t["top_val"].astype(np.float32), axis=1) <= 0).all()
    hid = np.load(os.path.join(HERE, "golden", "golden_hidden.npz"))["small_model"]
    assert np.array_equal(t["probe_hidden"].view(np.uint16), hid.view(np.uint16))
    import hashlib
    assert hashlib.sha256(logits.tobytes()).hexdigest() == g["last_logits_sha256"]
    # the weight directory holds exactly the reference's file set and sizes, and loads back
    d = str(tmp_path)
    orc.write_weight_dir(cfg, seed, d)
    names = sorted(os.listdir(d))
    assert len(names) == 13 * cfg.layers + 6
    H, I, V = cfg.hidden, cfg.inter, cfg.vocab
    assert os.path.getsize(os.path.join(d, "layer_0_wqkv.bin")) == 3 * H * H // 2
    assert os.path.getsize(os.path.join(d, "layer_0_bqkv_scale.bin")) == 2 * (3 * H // 128)
    assert os.path.getsize(os.path.join(d, "layer_3_w2.bin")) == H * I // 2
    assert os.path.getsize(os.path.join(d, "layer_3_w2_zp.bin")) == 2 * (H // 128)
    assert os.path.getsize(os.path.join(d, "word_embedding.bin")) == H * V // 2
    assert os.path.getsize(os.path.join(d, "unembed_scale.bin")) == 2 * (V // 128)
    assert os.path.getsize(os.path.join(d, "rms_norm_gamma_1.bin")) == 2 * H
    m2 = orc.Model(cfg)
    assert m2.load_dir(d) == 0
    ids2, _, _ = m2.generate(prompt, g["max_new"])
    assert np.array_equal(ids, ids2)
    os.remove(os.path.join(d, "layer_1_wo_zp.bin"))
    assert orc.Model(cfg).load_dir(d) != 0                      # missing file is an error
    with pytest.raises(ValueError):
        m.generate(np.arange(60, dtype=np.int32), 10)           # beyond max_pos


def test_reference_flow_versus_sample_first(orc):
    """Reference flow: decode step 0 feeds the last prompt token's final hidden state through the
    layers again (Inference.cu:1355-1363); sample_first samples before that pass.  Both flows are
    pinned; on the first step they see different hidden states, so their last-step logits differ."""
    a, b = GOLDEN["small_model"], GOLDEN["small_model_sample_first"]
    assert len(a["ids"]) == len(b["ids"]) == 10
    assert a["last_logits_sha256"] != b["last_logits_sha256"]
    assert a["ids"] != b["ids"]   # the seed was chosen so that the two flows are told apart by their ids as well
