"""ctypes binding of libqw3awq.so (include/qw3_cabi.h).

Thin by design: every function takes raw device pointers (ints) and a stream handle, exactly as
a C, C++ or FFI caller would.  There is no CPU fallback: if the library cannot be loaded, or a
call fails, an exception is raised.
"""
import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libqw3awq.so")
CSRC = os.path.join(_HERE, "csrc")

QW3_OK, QW3_ERR_ARG, QW3_ERR_CUDA, QW3_ERR_IO, QW3_ERR_RANGE = 0, 1, 2, 3, 4
QW3_ERR_TIMEOUT, QW3_ERR_DEVICE, QW3_ERR_NOMEM, QW3_ERR_STATE = 5, 6, 7, 8
EPI_STORE, EPI_RESIDUAL, EPI_GELU, EPI_ROPE_KV, EPI_ARGMAX = range(5)
MAX_STAGES = 8

# Every symbol include/qw3_cabi.h declares.
EXPORTS = [
    "qw3_strerror", "qw3_last_error", "qw3_dequant_w4", "qw3_w4_create", "qw3_w4_destroy", "qw3_ws_create",
    "qw3_ws_destroy", "qw3_ws_set_pdl", "qw3_ws_check", "qw3_gemv_w4a16", "qw3_gemv_w4a16_noalloc", "qw3_gemv_w4a16_noalloc_status", "qw3_gemm_w4a16", "qw3_rmsnorm",
    "qw3_rope_kv_append", "qw3_attn_decode", "qw3_attn_prefill", "qw3_handoff_wait", "qw3_embed_gather_w4", "qw3_argmax_f16", "qw3_config_default",
    "qw3_create", "qw3_destroy", "qw3_generate", "qw3_decode_more", "qw3_last_logits", "qw3_last_timing", "qw3_last_launches",
    "qw3_set_batched_prefill",
    "qw3_set_chained_decode",
    "qw3_kv_upload", "qw3_layer_decode", "qw3_stage_export", "qw3_stage_connect", "qw3_stage_layers",
    "qw3_fused_plan", "qw3_fused_repack_host", "qw3_stage_hidden", "qw3_tp_export", "qw3_tp_connect",
]


class Qw3Error(RuntimeError):
    def __init__(self, status, where, detail):
        super().__init__(f"{where}: status {status} ({detail})")
        self.status = status


class GemvArgs(C.Structure):
    _fields_ = [("d_x", C.c_void_p), ("d_gamma", C.c_void_p), ("eps", C.c_float), ("epilogue", C.c_int32),
                ("d_y", C.c_void_p), ("d_k_cache", C.c_void_p), ("d_v_cache", C.c_void_p), ("d_cos", C.c_void_p),
                ("d_sin", C.c_void_p), ("heads", C.c_int32), ("head_dim", C.c_int32), ("max_pos", C.c_int64),
                ("d_pos", C.c_void_p), ("pos", C.c_int32), ("d_token", C.c_void_p), ("d_logits_f32", C.c_void_p)]


class Config(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("inter", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
                ("layers", C.c_int32), ("vocab", C.c_int32), ("max_pos", C.c_int32), ("eps", C.c_float),
                ("rope_base", C.c_float), ("sample_first", C.c_int32), ("n_stages", C.c_int32),
                ("first_layer", C.c_int32 * (MAX_STAGES + 1)), ("device", C.c_int32 * MAX_STAGES),
                ("rank", C.c_int32), ("world", C.c_int32), ("use_graph", C.c_int32), ("use_pdl", C.c_int32),
                ("keep_logits", C.c_int32), ("persistent", C.c_int32), ("tensor_parallel", C.c_int32),
                ("attn_split_min", C.c_int32), ("cluster", C.c_int32)]


def build(force=False, verbose=False):
    """Compile the CUDA sources for sm_100a with the Makefile in csrc/ (nvcc cross-compiles on CPU)."""
    srcs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".cpp", ".h"))]
    srcs.append(os.path.join(_HERE, "..", "include", "qw3_cabi.h"))
    stale = not os.path.exists(LIB_PATH) or any(os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in srcs)
    if force or stale:
        cmd = ["make", "-C", CSRC, "-j8"] + (["-B"] if force else [])
        subprocess.check_call(cmd, stdout=None if verbose else subprocess.DEVNULL)
    return LIB_PATH


_lib = None


def lib():
    """Load the library (building it first if the sources are newer).  Raises if that fails."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        build()
    L = C.CDLL(LIB_PATH)
    vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int32, C.c_float
    L.qw3_strerror.restype = C.c_char_p
    L.qw3_strerror.argtypes = [C.c_int]
    L.qw3_last_error.restype = C.c_char_p
    L.qw3_last_error.argtypes = []
    sig = {
        "qw3_dequant_w4": [vp, vp, vp, i64, i64, i64, vp, vp],
        "qw3_w4_create": [vp, vp, vp, i64, i64, i64, C.c_int, C.POINTER(vp)],
        "qw3_w4_destroy": [vp],
        "qw3_ws_create": [C.POINTER(vp)],
        "qw3_ws_destroy": [vp],
        "qw3_ws_set_pdl": [vp, C.c_int],
        "qw3_ws_check": [vp, vp],
        "qw3_gemv_w4a16": [vp, C.POINTER(GemvArgs), vp, vp],
        "qw3_gemv_w4a16_noalloc": [vp, vp, vp, i64, i64, i64, C.c_int, vp, vp, vp],
        "qw3_gemv_w4a16_noalloc_status": [vp],
        "qw3_gemm_w4a16": [vp, vp, i64, vp, vp, vp],
        "qw3_rmsnorm": [vp, vp, i64, f32, vp, vp],
        "qw3_rope_kv_append": [vp, vp, vp, vp, vp, vp, i32, i32, i64, vp, i32, vp],
        "qw3_attn_decode": [vp, vp, vp, i32, i32, i64, vp, i32, vp, vp, vp],
        "qw3_attn_prefill": [vp, vp, vp, i32, i32, i64, i32, i32, vp, vp],
        "qw3_handoff_wait": [vp, i32, i64, i32, vp, vp],
        "qw3_embed_gather_w4": [vp, vp, vp, i64, i64, i64, vp, i32, vp, vp],
        "qw3_argmax_f16": [vp, i64, vp, vp, vp],
        "qw3_config_default": [C.POINTER(Config)],
        "qw3_create": [C.c_char_p, C.POINTER(Config), C.POINTER(vp)],
        "qw3_destroy": [vp],
        "qw3_generate": [vp, vp, i32, i32, vp, C.POINTER(i32)],
        "qw3_decode_more": [vp, i32, vp, C.POINTER(i32)],
        "qw3_last_logits": [vp, vp],
        "qw3_set_batched_prefill": [vp, i32],
        "qw3_set_chained_decode": [vp, i32],
        "qw3_last_timing": [vp, C.POINTER(f32), C.POINTER(f32)],
        "qw3_last_launches": [vp, C.POINTER(i64)],
        "qw3_kv_upload": [vp, i32, i32, vp, i64],
        "qw3_layer_decode": [vp, i32, i32, vp],
        "qw3_stage_export": [vp, vp],
        "qw3_stage_connect": [vp, vp, vp],
        "qw3_stage_layers": [C.POINTER(Config), i32, C.POINTER(i32), C.POINTER(i32)],
        "qw3_stage_hidden": [vp, i32, vp],
        "qw3_tp_export": [vp, vp],
        "qw3_tp_connect": [vp, vp],
        "qw3_fused_plan": [C.POINTER(Config), i32, i32, i32, vp, vp],
        "qw3_fused_repack_host": [C.POINTER(Config), i32, i32, i32, i32, vp, i64, vp, i64],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = C.c_int, args
    if hasattr(L, "qw3_debug_trace"):   # tracing builds only (make EXTRA=-DQW3_TRACE)
        L.qw3_debug_trace.restype, L.qw3_debug_trace.argtypes = C.c_int, [vp, i32, vp, i32, C.POINTER(i32)]
    _lib = L
    return L


def check(status, where):
    if status != QW3_OK:
        L = lib()
        raise Qw3Error(status, where, f"{L.qw3_strerror(status).decode()}; {L.qw3_last_error().decode()}")


def default_config(**kw):
    c = Config()
    check(lib().qw3_config_default(C.byref(c)), "qw3_config_default")
    for k, v in kw.items():
        if k in ("first_layer", "device"):
            for i, x in enumerate(v):
                getattr(c, k)[i] = x
        else:
            setattr(c, k, v)
    return c
