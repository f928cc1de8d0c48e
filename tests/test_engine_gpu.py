"""GPU parity of the engine (QWen3AWQInfer over the C ABI) against the CPU oracle: one decoder
layer, whole-model greedy decoding, stage-split invariance, error behaviour."""
import json
import os
import subprocess

import numpy as np
import pytest

from test_gemv_gpu import _ulp_diff

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "golden.json")))
GOLDEN_H = np.load(os.path.join(HERE, "golden", "golden_hidden.npz"))
SMALL = dict(hidden=512, inter=1536, heads=4, head_dim=128, layers=4, vocab=2176, max_pos=64, rope_base=10000.0)
SEED = GOLDEN["small_model"]["seed"]   # chosen so that the reference flow and sample_first give different ids


@pytest.fixture(scope="module")
def small_dir(orc, tmp_path_factory):
    d = str(tmp_path_factory.mktemp("w_small"))
    orc.write_weight_dir(orc.default_config(**SMALL), SEED, d)
    return d


def _oracle_generate(orc, cfg_kw, seed, weight_dir, prompt, max_new, sample_first=0):
    m = orc.Model(orc.default_config(sample_first=sample_first, **cfg_kw))
    assert m.load_dir(weight_dir) == 0
    out = m.generate(prompt, max_new)
    m.close()
    return out


def _logits_close(got32, want16):
    want = want16.astype(np.float32)
    return (np.abs(got32 - want) <= 2e-2 * np.abs(want) + 2e-2 * np.abs(want).mean()).all()


@pytest.mark.parametrize("persistent,use_graph,use_pdl", [(2, 0, 0), (2, 1, 0), (1, 0, 0), (1, 1, 0), (0, 0, 0), (0, 1, 0), (0, 0, 1), (0, 1, 1)])
def test_small_model_tokens_match_oracle(pkg, orc, cuda, small_dir, persistent, use_graph, use_pdl):
    prompt = orc.gen_tokens(SEED, orc.TOKENS, 6, SMALL["vocab"])
    ids, logits, margins = _oracle_generate(orc, SMALL, SEED, small_dir, prompt, 10)
    assert [int(t) for t in ids] == GOLDEN["small_model"]["ids"]          # the oracle itself is pinned
    inf = pkg.QWen3AWQInfer(small_dir, persistent=persistent, use_graph=use_graph, use_pdl=use_pdl, keep_logits=1, **SMALL)
    got = inf.generateResponse(prompt, 10)
    assert got == [int(t) for t in ids], f"margins {margins}"
    assert _logits_close(inf.last_logits(), logits)
    assert inf.generateResponse(prompt, 10) == got                         # the object is reusable
    assert inf.last_launches() > 0
    inf.close()


def test_small_model_batched_prefill(pkg, orc, cuda, small_dir):
    """Prompt in one block through the tensor-core contraction: same ids as the oracle's token loop, logits
    within the stated tolerance of it and of the token-at-a-time engine path."""
    prompt = orc.gen_tokens(SEED, orc.TOKENS, 6, SMALL["vocab"])
    ids, logits, margins = _oracle_generate(orc, SMALL, SEED, small_dir, prompt, 10)
    inf = pkg.QWen3AWQInfer(small_dir, keep_logits=1, **SMALL)
    loop_ids = inf.generateResponse(prompt, 10)
    loop_logits = inf.last_logits()
    inf.set_batched_prefill(True)
    got = inf.generateResponse(prompt, 10)
    assert got == [int(t) for t in ids] == loop_ids, f"margins {margins}"
    assert _logits_close(inf.last_logits(), logits)
    assert _logits_close(inf.last_logits(), loop_logits.astype(np.float16))
    inf.set_batched_prefill(False)
    assert inf.generateResponse(prompt, 10) == loop_ids                    # switching back restores the token loop
    inf.close()


@pytest.mark.parametrize("persistent", [2, 1, 0])
def test_small_model_sample_first(pkg, orc, cuda, small_dir, persistent):
    prompt = orc.gen_tokens(SEED, orc.TOKENS, 6, SMALL["vocab"])
    ids, _, _ = _oracle_generate(orc, SMALL, SEED, small_dir, prompt, 10, sample_first=1)
    assert [int(t) for t in ids] == GOLDEN["small_model_sample_first"]["ids"]
    assert GOLDEN["small_model_sample_first"]["ids"] != GOLDEN["small_model"]["ids"]   # the fixture can tell the two flows apart
    inf = pkg.QWen3AWQInfer(small_dir, sample_first=1, persistent=persistent, **SMALL)
    assert inf.generateResponse(prompt, 10) == [int(t) for t in ids]
    inf.close()


def _close(got, want, what):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    tol = 2e-2 * np.abs(want) + 2e-2 * np.abs(want).mean()
    assert (np.abs(got - want) <= tol).all(), f"{what}: max excess {(np.abs(got - want) - tol).max()}"


def _check_steps_and_probes(pkg, orc, name, wdir, cfg_kw, persistent, n_steps):
    """Per decode step: the sampled id, and the eight largest logits of the oracle within the stated tolerance (so a
    stale cache row or a position slip shows even where the arg-max would not move).  Hidden state after the first, a
    middle and the last layer at two positions, read at the boundaries of a three-stage split on one device."""
    g = GOLDEN[name]
    prompt = orc.gen_tokens(g["seed"], orc.TOKENS, g["n_prompt"], orc.default_config(**cfg_kw).vocab)
    assert [int(t) for t in prompt[:8]] == g["prompt_head"]
    inf = pkg.QWen3AWQInfer(wdir, keep_logits=1, persistent=persistent, sample_first=g["sample_first"], **cfg_kw)
    ids = []
    for step in range(n_steps):
        ids += inf.generateResponse(prompt, 1) if step == 0 else inf.decode_more(1)
        lg = inf.last_logits()
        assert ids[-1] == g["ids"][step], f"step {step}: margins {g['margins'][:n_steps]}"
        _close(lg[np.array(g["steps_top8_idx"][step])], g["steps_top8"][step], f"top-8 logits of step {step}")
    inf.close()
    if g["sample_first"]:
        return
    layers = g["probe_layers"]
    split = [0] + [l + 1 for l in layers]
    want = GOLDEN_H[name]
    inf = pkg.QWen3AWQInfer(wdir, n_stages=3, first_layer=split, device=[0, 0, 0], persistent=persistent, **cfg_kw)
    for pi, n_new in enumerate((0, g["probe_step"] + 1)):   # the last prompt token; the pass of decode step probe_step
        got_ids = inf.generateResponse(prompt, n_new)
        assert got_ids == g["ids"][:n_new]
        for k in range(3):
            _close(inf.stage_hidden(k), want[pi, k], f"hidden state after layer {layers[k]} at position {g['probe_pos'][pi]}")
    inf.close()


@pytest.mark.parametrize("persistent", [2, 1, 0])
@pytest.mark.parametrize("name", ["small_model", "small_model_sample_first"])
def test_small_model_every_step_and_hidden_probes(pkg, orc, cuda, small_dir, name, persistent):
    _check_steps_and_probes(pkg, orc, name, small_dir, SMALL, persistent, 10)


def test_small_model_attention_split_over_the_head_group(pkg, orc, cuda, small_dir):
    """The fused pass runs short contexts whole in every CTA of a head group and splits long ones over the group
    (attn_split_min); the default keeps the small model's contexts whole, so this run forces the split from the fourth
    position on: same ids, top-8 logits and hidden-state probes."""
    _check_steps_and_probes(pkg, orc, "small_model", small_dir, dict(SMALL, attn_split_min=3), 2, 10)


def test_small_model_head_groups_as_clusters(pkg, orc, cuda, small_dir):
    """cluster=1: on one GPU the CTAs of a head group form a thread-block cluster and exchange through distributed
    shared memory instead of tagged words in global memory (the default, and the form the row split over GPUs uses):
    same results, with the attention whole and split."""
    _check_steps_and_probes(pkg, orc, "small_model", small_dir, dict(SMALL, cluster=1), 2, 10)
    _check_steps_and_probes(pkg, orc, "small_model", small_dir, dict(SMALL, cluster=1, attn_split_min=3), 2, 10)


@pytest.mark.parametrize("persistent", [2, 1, 0])
@pytest.mark.parametrize("n_stages", [2, 3, 4])
def test_stage_split_does_not_change_tokens(pkg, orc, cuda, small_dir, n_stages, persistent):
    """Layer pipeline with several logical stages mapped onto one device: the hand-off is a local
    copy, the results must equal the single-stage run."""
    prompt = orc.gen_tokens(SEED, orc.TOKENS, 6, SMALL["vocab"])
    inf = pkg.QWen3AWQInfer(small_dir, n_stages=n_stages, device=[0] * n_stages, keep_logits=1, persistent=persistent, **SMALL)
    got = inf.generateResponse(prompt, 10)
    assert got == GOLDEN["small_model"]["ids"]
    _close(inf.last_logits()[np.array(GOLDEN["small_model"]["last_logits_top8_idx"])], GOLDEN["small_model"]["last_logits_top8"], "logits")
    inf.set_batched_prefill(True)       # the block of prompt rows is handed from stage to stage as well
    assert inf.generateResponse(prompt, 10) == GOLDEN["small_model"]["ids"]
    inf.close()


def test_one_decoder_layer_full_width(pkg, orc, cuda, tmp_path):
    """One Qwen3-8B-shape layer at batch 1: hidden 4096, 32 heads, wqkv 12288x4096, wo 4096x4096,
    w1/w2 at 12288, RoPE base 1e6, KV rows 0..511 pre-filled N(0,1), decode at position 512."""
    cfg_kw = dict(hidden=4096, inter=12288, heads=32, head_dim=128, layers=1, vocab=1024, max_pos=1024, rope_base=1e6)
    d = str(tmp_path)
    cfg = orc.default_config(**cfg_kw)
    orc.write_weight_dir(cfg, 0, d)
    m = orc.Model(cfg)
    assert m.load_dir(d) == 0
    m.fill_kv(0, 512)
    hidden = orc.gen_normal_f16(0, orc.ACT, 4096)
    want = m.layer(0, 512, hidden)
    inf = pkg.QWen3AWQInfer(d, **cfg_kw)
    for which in (0, 1):
        kv = m.kv(0, which).reshape(32, 1024, 128)[:, :512].copy()
        inf.kv_upload(0, which, kv, 512)
    got = inf.layer_decode(0, 512, hidden)
    inf.close()
    m.close()
    err = np.abs(got.astype(np.float32) - want.astype(np.float32))
    assert (err <= 2e-2 * np.abs(want.astype(np.float32)) + 2e-2 * np.abs(want.astype(np.float32)).mean()).all()
    d_ulp = _ulp_diff(got, want)
    assert (d_ulp > 1).mean() < 0.02, f"{(d_ulp > 1).mean():.4f} of the hidden state is more than one ulp off"


@pytest.fixture(scope="module")
def full_dir(orc, tmp_path_factory):
    d = str(tmp_path_factory.mktemp("w_full"))
    orc.write_weight_dir(orc.default_config(), GOLDEN["full_model"]["seed"], d)
    return d


def test_full_model_tokens_match_golden(pkg, orc, cuda, full_dir):
    """Full 36-layer model, prompt 128, 72 greedy tokens, one GPU; expected ids were produced by the
    CPU oracle (tests/golden/make_golden.py --full) from the same seeded weights."""
    g = GOLDEN["full_model"]
    cfg = orc.default_config(**g["config"])
    prompt = orc.gen_tokens(g["seed"], orc.TOKENS, g["n_prompt"], cfg.vocab)
    assert [int(t) for t in prompt[:8]] == g["prompt_head"]
    inf = pkg.QWen3AWQInfer(full_dir, keep_logits=1, **g["config"])
    inf.set_batched_prefill(False)      # the reference's token loop (a new object would take blocks for this prompt length)
    got = inf.generateResponse(prompt, g["max_new"])
    logits = inf.last_logits()
    # the same run with the prompt as one block of 128 rows through the tensor-core contraction
    inf.set_batched_prefill(True)
    got_b = inf.generateResponse(prompt, g["max_new"])
    logits_b = inf.last_logits()
    prompt_ms_b = inf.last_timing()[0]
    inf.close()
    assert got == g["ids"], f"oracle top-1/top-2 margins per step: {g['margins']}"
    top = np.array(g["last_logits_top8_idx"])
    _close(logits[top], g["last_logits_top8"], "last-step logits")
    assert got_b == g["ids"], f"batched prompt phase; margins {g['margins']}"
    _close(logits_b[top], g["last_logits_top8"], "last-step logits, batched prompt phase")
    assert prompt_ms_b > 0


@pytest.mark.parametrize("persistent", [2, 1])
def test_full_model_every_step_and_hidden_probes(pkg, orc, cuda, full_dir, persistent):
    """The 36-layer model step by step: ids, top-8 logits of every step, hidden state after layers 0, 17 and 35 at the
    last prompt position and at decode step 19."""
    _check_steps_and_probes(pkg, orc, "full_model", full_dir, GOLDEN["full_model"]["config"], persistent, 24)


def test_full_model_head_groups_as_clusters(pkg, orc, cuda, full_dir):
    """The same 24 steps and probes with the head groups as thread-block clusters (what bench.py runs on one GPU)."""
    _check_steps_and_probes(pkg, orc, "full_model", full_dir, dict(GOLDEN["full_model"]["config"], cluster=1), 2, 24)


def test_errors_are_status_codes(pkg, orc, cuda, small_dir, tmp_path):
    cabi = pkg.cabi
    with pytest.raises(cabi.Qw3Error) as e:   # missing directory
        pkg.QWen3AWQInfer(str(tmp_path / "nowhere"), **SMALL)
    assert e.value.status == cabi.QW3_ERR_IO
    d = str(tmp_path / "short")
    subprocess.check_call(["cp", "-r", small_dir, d])
    with open(os.path.join(d, "layer_2_w1.bin"), "r+b") as f:   # short file (Inference.cu:305-308)
        f.truncate(100)
    with pytest.raises(cabi.Qw3Error) as e:
        pkg.QWen3AWQInfer(d, **SMALL)
    assert e.value.status == cabi.QW3_ERR_IO
    with pytest.raises(cabi.Qw3Error) as e:   # more stages than devices
        pkg.QWen3AWQInfer(small_dir, n_stages=2, device=[0, 99], **SMALL)
    assert e.value.status == cabi.QW3_ERR_DEVICE
    inf = pkg.QWen3AWQInfer(small_dir, **SMALL)
    with pytest.raises(cabi.Qw3Error) as e:   # prompt + new tokens beyond the KV capacity
        inf.generateResponse([1] * 60, 10)
    assert e.value.status == cabi.QW3_ERR_RANGE
    with pytest.raises(cabi.Qw3Error) as e:   # token id outside the vocabulary
        inf.generateResponse([5, 999999], 2)
    assert e.value.status == cabi.QW3_ERR_RANGE
    with pytest.raises(cabi.Qw3Error) as e:   # empty prompt
        inf.generateResponse([], 2)
    assert e.value.status == cabi.QW3_ERR_RANGE
    assert inf.generateResponse([5, 6], 0) == []
    assert len(inf.generateResponse([5, 6], 3)) == 3            # still usable after the errors
    inf.close()


def test_example_binary_prints_oracle_tokens(pkg, orc, cuda, small_dir):
    """The reference's main (Inference.cu:1413-1433): single-token prompt, 20 new tokens."""
    exe = os.path.join(os.path.dirname(pkg.cabi.LIB_PATH), "qwen3_awq_infer")
    out = subprocess.run([exe, small_dir, "20", "1", "4", "512", "1536", "2176", "64"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    ids, _, _ = _oracle_generate(orc, SMALL, SEED, small_dir, np.array([0], np.int32), 20)
    assert out.stdout.split(":")[1].split() == [str(int(t)) for t in ids]
