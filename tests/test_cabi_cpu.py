"""CPU checks of the boundary: the C-ABI library builds for sm_100a, loads without a GPU, exports
every symbol the header declares, and rejects bad input with status codes (no compute calls)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(pkg):
    cabi = pkg.cabi
    cabi.build()
    L = cabi.lib()
    header = open(os.path.join(ROOT, "include", "qw3_cabi.h")).read()
    header = re.sub(r"#ifdef QW3_TRACE.*?#endif", "", header, flags=re.S)   # declared in tracing builds of the library only
    declared = set(re.findall(r"\b(qw3_[a-z0-9_]+)\s*\(", header))
    assert declared == set(cabi.EXPORTS), declared ^ set(cabi.EXPORTS)
    for name in declared:
        assert hasattr(L, name), name


def test_status_strings_and_default_config(pkg):
    cabi = pkg.cabi
    L = cabi.lib()
    assert L.qw3_strerror(0) == b"ok"
    assert b"KV" in L.qw3_strerror(cabi.QW3_ERR_RANGE)
    c = cabi.default_config()
    # Inference.cu:33-47
    assert (c.hidden, c.inter, c.heads, c.head_dim, c.layers, c.vocab, c.max_pos) == (4096, 12288, 32, 128, 36, 151936, 40960)
    assert abs(c.eps - 1e-6) < 1e-12 and c.rope_base == 10000.0 and c.sample_first == 0
    assert c.n_stages == 1 and c.world == 1 and c.rank == 0


def test_config_struct_matches_the_header(pkg):
    cabi = pkg.cabi
    header = open(os.path.join(ROOT, "include", "qw3_cabi.h")).read()
    body = header[header.index("typedef struct Qw3Config {"):header.index("} Qw3Config;")]
    fields = re.findall(r"^\s*(?:int32_t|float)\s+([a-z_]+)(?:\[[^\]]+\])?;", body, re.M)
    assert fields == [f[0] for f in cabi.Config._fields_]
    body = header[header.index("typedef struct Qw3GemvArgs {"):header.index("} Qw3GemvArgs;")]
    fields = re.findall(r"^\s*(?:const\s+)?(?:void|int32_t|int64_t|float)\s*\*?\s+([a-z_0-9]+);", body, re.M)
    assert fields == [f[0] for f in cabi.GemvArgs._fields_]


def test_bad_configuration_is_rejected_without_a_gpu(pkg, tmp_path):
    cabi = pkg.cabi
    L = cabi.lib()
    h = C.c_void_p()
    for kw in (dict(head_dim=64), dict(hidden=4000), dict(n_stages=9), dict(n_stages=0), dict(vocab=1000),
               dict(n_stages=2, first_layer=[0, 0, 36]), dict(world=2, rank=2)):
        cfg = cabi.default_config(**kw)
        assert L.qw3_create(str(tmp_path).encode(), C.byref(cfg), C.byref(h)) == cabi.QW3_ERR_ARG, kw
        assert L.qw3_last_error() != b""
    assert L.qw3_create(None, None, C.byref(h)) == cabi.QW3_ERR_ARG


def test_null_arguments_are_rejected_without_a_gpu(pkg):
    cabi = pkg.cabi
    L = cabi.lib()
    assert L.qw3_dequant_w4(None, None, None, 1, 1, 1, None, None) == cabi.QW3_ERR_ARG
    assert L.qw3_w4_create(None, None, None, 1, 128, 128, 1, None) == cabi.QW3_ERR_ARG
    assert L.qw3_gemv_w4a16(None, None, None, None) == cabi.QW3_ERR_ARG
    assert L.qw3_rmsnorm(None, None, 0, 1e-6, None, None) == cabi.QW3_ERR_ARG
    assert L.qw3_attn_decode(None, None, None, 32, 128, 64, None, 0, None, None, None) == cabi.QW3_ERR_ARG
    assert L.qw3_argmax_f16(None, 10, None, None, None) == cabi.QW3_ERR_ARG
    assert L.qw3_generate(None, None, 0, 0, None, None) == cabi.QW3_ERR_ARG
    assert L.qw3_destroy(None) == cabi.QW3_OK


def test_product_code_does_not_reach_the_oracle():
    """Nothing in the package or the headers may import, link or name the oracle."""
    pkg_dir = os.path.join(ROOT, "cuda-kernel-qwen3-8b-awq_b200")
    for base, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", "Makefile")):
                text = open(os.path.join(base, f), errors="ignore").read()
                assert "oracle" not in text.lower() and "orc." not in text, os.path.join(base, f)
