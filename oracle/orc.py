"""ctypes binding of the CPU oracle (oracle/qw3_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the bench's CPU-baseline
leg, never by the shipped library.  PARITY UNPINNED (the reference has no golden vectors and no
CPU path); see qw3_oracle.h.  fp16 data crosses as numpy uint16/float16 arrays.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqw3_oracle.so")

# enum OrcKind
WQKV, WQKV_SCALE, WQKV_ZP, WO, WO_SCALE, WO_ZP, W1, W1_SCALE, W1_ZP, W2, W2_SCALE, W2_ZP = range(12)
GAMMA, EMB, EMB_SCALE, EMB_ZP, UNEMB, UNEMB_SCALE, UNEMB_ZP, ACT, KV_K, KV_V, TOKENS = range(12, 23)


class OrcConfig(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("inter", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
                ("layers", C.c_int32), ("vocab", C.c_int32), ("max_pos", C.c_int32), ("group", C.c_int32),
                ("eps", C.c_float), ("rope_base", C.c_float), ("sample_first", C.c_int32)]


def build(force=False):
    """Compile the oracle with the Makefile beside it (g++ only)."""
    src = [os.path.join(_HERE, f) for f in ("qw3_oracle.cpp", "qw3_oracle.h")]
    stale = not os.path.exists(_LIB_PATH) or any(os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "libqw3_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(_LIB_PATH)
    u64, i64, i32, vp, dbl, flt = C.c_uint64, C.c_int64, C.c_int32, C.c_void_p, C.c_double, C.c_float
    sig = {
        "orc_mix64": (u64, [u64]),
        "orc_stream_key": (u64, [u64, u64]),
        "orc_gen_codes": (None, [u64, u64, i64, vp]),
        "orc_gen_normal_f16": (None, [u64, u64, i64, dbl, dbl, i32, vp]),
        "orc_gen_uniform_int_f16": (None, [u64, u64, i64, i32, i32, vp]),
        "orc_gen_tokens": (None, [u64, u64, i64, i32, vp]),
        "orc_dequant": (None, [vp, vp, vp, i64, i64, i64, i32, vp]),
        "orc_gemm_w4a16": (None, [vp, vp, vp, i64, i64, i64, i32, vp, i64, i32, vp, vp]),
        "orc_rmsnorm": (None, [vp, vp, i64, flt, vp]),
        "orc_rope_tables": (None, [i32, i32, flt, vp, vp]),
        "orc_rope": (None, [vp, i32, i32, vp, vp, i32]),
        "orc_attention": (None, [vp, vp, vp, i32, i32, i64, i64, vp]),
        "orc_gelu": (None, [vp, i64]),
        "orc_add": (None, [vp, vp, i64, vp]),
        "orc_argmax_f16": (i64, [vp, i64]),
        "orc_embed_gather": (None, [vp, vp, vp, i64, i64, i64, i32, i64, vp]),
        "orc_config_default": (None, [C.POINTER(OrcConfig)]),
        "orc_model_new": (vp, [C.POINTER(OrcConfig)]),
        "orc_model_free": (None, [vp]),
        "orc_model_init_random": (i32, [vp, u64]),
        "orc_model_load_dir": (i32, [vp, C.c_char_p]),
        "orc_write_weight_dir": (i32, [C.POINTER(OrcConfig), u64, C.c_char_p]),
        "orc_model_fill_kv": (None, [vp, u64, i64]),
        "orc_model_layer": (None, [vp, i32, i64, vp]),
        "orc_model_sample": (i64, [vp, vp, vp]),
        "orc_model_generate": (i32, [vp, vp, i32, i32, vp, vp, vp]),
        "orc_model_generate_trace": (i32, [vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, i32, vp, i32, vp]),
        "orc_model_packed": (vp, [vp, i32, i32]),
        "orc_model_f16": (vp, [vp, i32, i32]),
        "orc_model_kv": (vp, [vp, i32, i32]),
        "orc_num_threads": (i32, []),
        "orc_set_num_threads": (None, [i32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _lib = L
    return L


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def default_config(**kw):
    c = OrcConfig()
    lib().orc_config_default(C.byref(c))
    for k, v in kw.items():
        setattr(c, k, v)
    return c


# ---- generator -------------------------------------------------------------------------------
def gen_codes(seed, tag, n_bytes):
    out = np.empty(n_bytes, np.uint8)
    lib().orc_gen_codes(seed, tag, n_bytes, _p(out))
    return out


def gen_normal_f16(seed, tag, n, mean=0.0, std=1.0, take_abs=False):
    out = np.empty(n, np.float16)
    lib().orc_gen_normal_f16(seed, tag, n, mean, std, int(take_abs), _p(out))
    return out


def gen_uniform_int_f16(seed, tag, n, lo, hi):
    out = np.empty(n, np.float16)
    lib().orc_gen_uniform_int_f16(seed, tag, n, lo, hi, _p(out))
    return out


def gen_tokens(seed, tag, n, vocab):
    out = np.empty(n, np.int32)
    lib().orc_gen_tokens(seed, tag, n, vocab, _p(out))
    return out


def gen_linear(seed, out_dim, in_dim, layer=0, kind=WQKV, group=128):
    """One AWQ linear in the reference's on-disk form: packed bytes, scale and zero-point with
    out_dim/group entries each (scale |N(0,1)|*0.02, zero-point uniform integer 6..9)."""
    packed = gen_codes(seed, layer * 64 + kind, out_dim * ((in_dim + 1) // 2))
    scale = gen_normal_f16(seed, layer * 64 + kind + 1, out_dim // group, 0.0, 0.02, True)
    zp = gen_uniform_int_f16(seed, layer * 64 + kind + 2, out_dim // group, 6, 9)
    return packed, scale, zp


# ---- operators -------------------------------------------------------------------------------
def dequant(packed, scale, zp, rows, cols, group=128):
    out = np.empty((rows, cols), np.float16)
    lib().orc_dequant(_p(packed), _p(scale), _p(zp), scale.size, rows, cols, group, _p(out))
    return out


def gemm_w4a16(packed, scale, zp, M, K, x, group=128, acc64=True):
    """x: float16 [K] or [R, K].  Returns (y_f32, y_f16) shaped like x with K replaced by M."""
    x2 = np.ascontiguousarray(x.reshape(-1, K))
    R = x2.shape[0]
    y32 = np.empty((R, M), np.float32)
    y16 = np.empty((R, M), np.float16)
    lib().orc_gemm_w4a16(_p(packed), _p(scale), _p(zp), scale.size, M, K, group, _p(x2), R, int(acc64), _p(y32), _p(y16))
    if x.ndim == 1:
        return y32[0], y16[0]
    return y32, y16


def rmsnorm(x, gamma, eps=1e-6):
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(gamma), x.size, eps, _p(out))
    return out


def rope_tables(max_pos, head_dim, base):
    cos_t = np.empty((max_pos, head_dim // 2), np.float16)
    sin_t = np.empty((max_pos, head_dim // 2), np.float16)
    lib().orc_rope_tables(max_pos, head_dim, base, _p(cos_t), _p(sin_t))
    return cos_t, sin_t


def rope(qk, heads, head_dim, cos_t, sin_t, pos):
    out = np.ascontiguousarray(qk).copy()
    lib().orc_rope(_p(out), heads, head_dim, _p(cos_t), _p(sin_t), pos)
    return out


def attention(q, k_cache, v_cache, heads, head_dim, max_pos, length):
    ctx = np.empty(heads * head_dim, np.float16)
    lib().orc_attention(_p(q), _p(k_cache), _p(v_cache), heads, head_dim, max_pos, length, _p(ctx))
    return ctx


def gelu(x):
    out = np.ascontiguousarray(x).copy()
    lib().orc_gelu(_p(out), out.size)
    return out


def add(a, b):
    out = np.empty_like(a)
    lib().orc_add(_p(a), _p(b), a.size, _p(out))
    return out


def argmax_f16(logits):
    return int(lib().orc_argmax_f16(_p(logits), logits.size))


def embed_gather(packed, scale, zp, hidden, vocab, tok, group=128):
    out = np.empty(hidden, np.float16)
    lib().orc_embed_gather(_p(packed), _p(scale), _p(zp), scale.size, hidden, vocab, group, tok, _p(out))
    return out


# ---- model -----------------------------------------------------------------------------------
class Model:
    def __init__(self, cfg):
        self.cfg = cfg
        self.h = lib().orc_model_new(C.byref(cfg))

    def close(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def init_random(self, seed):
        assert lib().orc_model_init_random(self.h, seed) == 0

    def load_dir(self, path):
        return lib().orc_model_load_dir(self.h, path.encode())

    def fill_kv(self, seed, upto):
        lib().orc_model_fill_kv(self.h, seed, upto)

    def layer(self, layer, pos, hidden):
        h = np.ascontiguousarray(hidden).copy()
        lib().orc_model_layer(self.h, layer, pos, _p(h))
        return h

    def sample(self, hidden):
        logits = np.empty(self.cfg.vocab, np.float16)
        tok = lib().orc_model_sample(self.h, _p(hidden), _p(logits))
        return int(tok), logits

    def generate(self, prompt, max_new):
        prompt = np.ascontiguousarray(prompt, np.int32)
        ids = np.empty(max_new, np.int32)
        logits = np.empty(self.cfg.vocab, np.float16)
        margins = np.empty(max_new, np.float32)
        rc = lib().orc_model_generate(self.h, _p(prompt), prompt.size, max_new, _p(ids), _p(logits), _p(margins))
        if rc != 0:
            raise ValueError("oracle: invalid prompt/max_new for this configuration")
        return ids, logits, margins

    def generate_trace(self, prompt, max_new, probe_layers=(), probe_pos=()):
        """generate() with probes: returns a dict with ids, last logits, margins, per-step top-8 (idx, val) and the
        hidden state after probe_layers at probe_pos ([n_pos][n_layers][hidden] fp16)."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        ids = np.empty(max_new, np.int32)
        logits = np.empty(self.cfg.vocab, np.float16)
        margins = np.empty(max_new, np.float32)
        top_idx = np.empty((max_new, 8), np.int32)
        top_val = np.empty((max_new, 8), np.float16)
        pl = np.ascontiguousarray(probe_layers, np.int32)
        pp = np.ascontiguousarray(probe_pos, np.int32)
        ph = np.zeros((pp.size, pl.size, self.cfg.hidden), np.float16)
        rc = lib().orc_model_generate_trace(self.h, _p(prompt), prompt.size, max_new, _p(ids), _p(logits), _p(margins),
                                            _p(top_idx), _p(top_val), _p(pl) if pl.size else None, pl.size,
                                            _p(pp) if pp.size else None, pp.size, _p(ph) if ph.size else None)
        if rc != 0:
            raise ValueError("oracle: invalid prompt/max_new for this configuration")
        return dict(ids=ids, logits=logits, margins=margins, top_idx=top_idx, top_val=top_val, probe_hidden=ph)

    def _view(self, ptr, n, dtype):
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(n * np.dtype(dtype).itemsize,)).view(dtype)

    def packed(self, layer, kind, n_bytes):
        return self._view(lib().orc_model_packed(self.h, layer, kind), n_bytes, np.uint8)

    def f16(self, layer, kind, n):
        return self._view(lib().orc_model_f16(self.h, layer, kind), n, np.float16)

    def kv(self, layer, which):
        c = self.cfg
        return self._view(lib().orc_model_kv(self.h, layer, which), c.heads * c.max_pos * c.head_dim, np.float16)


def write_weight_dir(cfg, seed, path):
    os.makedirs(path, exist_ok=True)
    if lib().orc_write_weight_dir(C.byref(cfg), seed, path.encode()) != 0:
        raise OSError("oracle: could not write weight dir " + path)


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(n):
    lib().orc_set_num_threads(int(n))
