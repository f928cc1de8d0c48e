"""Regenerates tests/golden/golden.json from the CPU oracle (oracle/qw3_oracle.cpp).

    python tests/golden/make_golden.py [--full]

The reference ships no golden vectors (it has no tests and does not build), so these fixtures pin
the oracle and the seeded generator against silent change, and let the GPU tests check the
full-size configurations without re-running minutes of CPU work.  --full also runs the 36-layer
configuration (prompt 128 + 20 tokens; a few minutes on 8 cores); without it the entry already in
golden.json is kept.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import orc  # noqa: E402

OUT = os.path.join(HERE, "golden.json")

SMALL = dict(hidden=512, inter=1536, heads=4, head_dim=128, layers=4, vocab=2176, max_pos=64, rope_base=10000.0)
FULL = dict(max_pos=256)   # reference constants otherwise; KV rows kept = 256 >= 128 + 20


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def model_case(cfg_kw, seed, n_prompt, max_new, sample_first=0):
    cfg = orc.default_config(sample_first=sample_first, **cfg_kw)
    m = orc.Model(cfg)
    m.init_random(seed)
    prompt = orc.gen_tokens(seed, orc.TOKENS, n_prompt, cfg.vocab)
    ids, logits, margins = m.generate(prompt, max_new)
    top = np.argsort(-logits.astype(np.float32), kind="stable")[:8]
    case = dict(config=cfg_kw, seed=seed, n_prompt=n_prompt, max_new=max_new, sample_first=sample_first,
                prompt_head=[int(t) for t in prompt[:8]], ids=[int(t) for t in ids],
                min_margin=float(margins.min()), margins=[float(x) for x in margins],
                last_logits_sha256=sha(logits), last_logits_top8_idx=[int(t) for t in top],
                last_logits_top8=[float(logits[t]) for t in top])
    m.close()
    return case


def main():
    full = "--full" in sys.argv
    old = json.load(open(OUT)) if os.path.exists(OUT) else {}
    g = {}
    # generator pins
    g["generator"] = dict(
        codes_seed0_tag0=orc.gen_codes(0, 0, 32).tobytes().hex(),
        scale_seed0_tag1=orc.gen_normal_f16(0, 1, 8, 0.0, 0.02, True).tobytes().hex(),
        zp_seed0_tag2=orc.gen_uniform_int_f16(0, 2, 8, 6, 9).tobytes().hex(),
        act_seed0=orc.gen_normal_f16(0, orc.ACT, 8).tobytes().hex(),
        tokens_seed0=[int(t) for t in orc.gen_tokens(0, orc.TOKENS, 8, 151936)],
    )
    # single AWQ linear, seed 0: 4096 x 4096
    M = K = 4096
    p, s, z = orc.gen_linear(0, M, K)
    x = orc.gen_normal_f16(0, orc.ACT, K)
    dq = orc.dequant(p, s, z, M, K)
    y32, y16 = orc.gemm_w4a16(p, s, z, M, K, x)
    g["single_linear"] = dict(M=M, K=K, seed=0, packed_sha256=sha(p), dequant_sha256=sha(dq), y_f16_sha256=sha(y16),
                              y_f16_head=y16[:8].tobytes().hex(), y_f32_head=[float(v) for v in y32[:8]])
    g["small_model"] = model_case(SMALL, 0, 6, 10)
    g["small_model_sample_first"] = model_case(SMALL, 0, 6, 10, sample_first=1)
    if full:
        g["full_model"] = model_case(FULL, 0, 128, 20)
    elif "full_model" in old:
        g["full_model"] = old["full_model"]
    json.dump(g, open(OUT, "w"), indent=1)
    print("wrote", OUT, "full" if full else "(full-size entry kept)")


if __name__ == "__main__":
    main()
