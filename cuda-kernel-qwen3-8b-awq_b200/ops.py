"""Per-operator entry points of the C ABI on torch CUDA tensors.

torch is used for device memory and streams only; every operator runs in libqw3awq.so.  fp16
tensors are torch.float16; packed weights are torch.uint8.
"""
import ctypes as C

import torch

from . import cabi


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class Workspace:
    def __init__(self, pdl=False):
        self.h = C.c_void_p()
        cabi.check(cabi.lib().qw3_ws_create(C.byref(self.h)), "qw3_ws_create")
        cabi.check(cabi.lib().qw3_ws_set_pdl(self.h, int(pdl)), "qw3_ws_set_pdl")

    def check(self):
        cabi.check(cabi.lib().qw3_ws_check(self.h, _stream()), "qw3_ws_check")

    def close(self):
        if self.h.value:
            cabi.lib().qw3_ws_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class W4Linear:
    """One AWQ matrix in the on-disk layout, resident on the GPU (AWQWeight without d_dq)."""

    def __init__(self, packed, scale, zp, out_dim, in_dim, zp_integral=True):
        self.packed, self.scale, self.zp = packed, scale, zp   # keep the tensors alive
        self.out_dim, self.in_dim = out_dim, in_dim
        self.h = C.c_void_p()
        cabi.check(cabi.lib().qw3_w4_create(_ptr(packed), _ptr(scale), _ptr(zp), scale.numel(), out_dim, in_dim,
                                            int(zp_integral), C.byref(self.h)), "qw3_w4_create")

    def close(self):
        if self.h.value:
            cabi.lib().qw3_w4_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def dequant_w4(packed, scale, zp, rows, cols):
    out = torch.empty((rows, cols), dtype=torch.float16, device=packed.device)
    cabi.check(cabi.lib().qw3_dequant_w4(_ptr(packed), _ptr(scale), _ptr(zp), scale.numel(), rows, cols, _ptr(out), _stream()),
               "qw3_dequant_w4")
    return out


def gemv_args(x, epilogue=cabi.EPI_STORE, y=None, gamma=None, eps=1e-6, k_cache=None, v_cache=None, cos=None, sin=None,
              heads=0, max_pos=0, d_pos=None, pos=0, d_token=None, logits_f32=None):
    a = cabi.GemvArgs()
    a.d_x, a.d_gamma, a.eps, a.epilogue, a.d_y = _ptr(x), _ptr(gamma), eps, epilogue, _ptr(y)
    a.d_k_cache, a.d_v_cache, a.d_cos, a.d_sin = _ptr(k_cache), _ptr(v_cache), _ptr(cos), _ptr(sin)
    a.heads, a.head_dim, a.max_pos, a.d_pos, a.pos = heads, 128, max_pos, _ptr(d_pos), pos
    a.d_token, a.d_logits_f32 = _ptr(d_token), _ptr(logits_f32)
    return a


def gemv_w4a16(w, ws, args):
    cabi.check(cabi.lib().qw3_gemv_w4a16(w.h, C.byref(args), ws.h, _stream()), "qw3_gemv_w4a16")


def gemm_w4a16(w, ws, x, y):
    cabi.check(cabi.lib().qw3_gemm_w4a16(w.h, _ptr(x), x.shape[0], _ptr(y), ws.h, _stream()), "qw3_gemm_w4a16")


def rmsnorm(x, gamma, eps=1e-6):
    out = torch.empty_like(x)
    cabi.check(cabi.lib().qw3_rmsnorm(_ptr(x), _ptr(gamma), x.numel(), eps, _ptr(out), _stream()), "qw3_rmsnorm")
    return out


def rope_kv_append(qkv, q_out, k_cache, v_cache, cos, sin, heads, max_pos, pos, d_pos=None):
    cabi.check(cabi.lib().qw3_rope_kv_append(_ptr(qkv), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(cos), _ptr(sin),
                                             heads, 128, max_pos, _ptr(d_pos), pos, _stream()), "qw3_rope_kv_append")


def attn_decode(q, k_cache, v_cache, heads, max_pos, pos, ws, d_pos=None):
    ctx = torch.empty(heads * 128, dtype=torch.float16, device=q.device)
    cabi.check(cabi.lib().qw3_attn_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), heads, 128, max_pos, _ptr(d_pos), pos,
                                          _ptr(ctx), ws.h, _stream()), "qw3_attn_decode")
    return ctx


def attn_prefill(qkv, k_cache, v_cache, heads, max_pos, pos0, rows):
    """Causal attention of a block of prompt rows (qkv: [rows][3 * heads * 128], q already rotated)."""
    ctx = torch.empty(rows, heads * 128, dtype=torch.float16, device=qkv.device)
    cabi.check(cabi.lib().qw3_attn_prefill(_ptr(qkv), _ptr(k_cache), _ptr(v_cache), heads, 128, max_pos, pos0, rows, _ptr(ctx),
                                           _stream()), "qw3_attn_prefill")
    return ctx


def embed_gather_w4(packed, scale, zp, hidden, vocab, token, d_token=None):
    out = torch.empty(hidden, dtype=torch.float16, device=packed.device)
    cabi.check(cabi.lib().qw3_embed_gather_w4(_ptr(packed), _ptr(scale), _ptr(zp), scale.numel(), hidden, vocab,
                                              _ptr(d_token), token, _ptr(out), _stream()), "qw3_embed_gather_w4")
    return out


def argmax_f16(logits, ws):
    tok = torch.zeros(1, dtype=torch.int32, device=logits.device)
    cabi.check(cabi.lib().qw3_argmax_f16(_ptr(logits), logits.numel(), _ptr(tok), ws.h, _stream()), "qw3_argmax_f16")
    return tok
