"""QWen3AWQInfer: the reference's public class (Inference.cu:356-366) over the C ABI.

Same two calls -- construct from a weight directory, generateResponse(prompt_ids, max_new_tokens)
returning only the new ids -- with errors raised as exceptions instead of std::exit(1)
(Inference.cu:52-71).  All compute happens in libqw3awq.so on the GPU; nothing here falls back
to the CPU.
"""
import ctypes as C

from . import cabi


class QWen3AWQInfer:
    def __init__(self, weight_dir, config=None, **overrides):
        """weight_dir holds the raw .bin files named as in Inference.cu:780-900.  `config` is a
        cabi.Config (default: the reference constants, Inference.cu:33-47, on one GPU); keyword
        overrides set single fields, e.g. n_stages=2, device=[0, 1], rope_base=1e6."""
        self._lib = cabi.lib()
        self.config = config if config is not None else cabi.default_config()
        for k, v in overrides.items():
            if k in ("first_layer", "device"):
                for i, x in enumerate(v):
                    getattr(self.config, k)[i] = x
            else:
                setattr(self.config, k, v)
        self._h = C.c_void_p()
        cabi.check(self._lib.qw3_create(str(weight_dir).encode(), C.byref(self.config), C.byref(self._h)), "qw3_create")

    def generateResponse(self, prompt_ids, max_new_tokens):
        """Inference.cu:1297-1408: feeds the prompt token by token, then returns max_new_tokens
        greedy ids."""
        n = len(prompt_ids)
        prompt = (C.c_int32 * max(n, 1))(*[int(t) for t in prompt_ids])
        out = (C.c_int32 * max(max_new_tokens, 1))()
        n_out = C.c_int32(0)
        cabi.check(self._lib.qw3_generate(self._h, prompt, n, max_new_tokens, out, C.byref(n_out)), "qw3_generate")
        return [int(out[i]) for i in range(n_out.value)]

    def set_batched_prefill(self, on):
        """Prompt in blocks of rows through the tensor-core contraction (True), token by token as the reference
        (False), or None: blocks for prompts of 16 tokens or more (the default of a new object)."""
        cabi.check(self._lib.qw3_set_batched_prefill(self._h, -1 if on is None else (1 if on else 0)), "qw3_set_batched_prefill")

    def set_chained_decode(self, on):
        """One process per GPU: chain the stages inside the token-pass kernels from the second decode step on (True,
        the default) or keep the mailbox send / receive launches for every step (False).  Set every stage alike."""
        cabi.check(self._lib.qw3_set_chained_decode(self._h, 1 if on else 0), "qw3_set_chained_decode")

    def decode_more(self, max_new_tokens):
        """Continue the last generateResponse call for max_new_tokens more ids (same KV state)."""
        out = (C.c_int32 * max(max_new_tokens, 1))()
        n_out = C.c_int32(0)
        cabi.check(self._lib.qw3_decode_more(self._h, max_new_tokens, out, C.byref(n_out)), "qw3_decode_more")
        return [int(out[i]) for i in range(n_out.value)]

    def last_logits(self):
        """fp32 logits of the last decode step (needs keep_logits=1)."""
        import numpy as np
        out = np.empty(self.config.vocab, np.float32)
        cabi.check(self._lib.qw3_last_logits(self._h, out.ctypes.data_as(C.c_void_p)), "qw3_last_logits")
        return out

    def last_timing(self):
        """(prompt_ms, decode_ms) of the last generateResponse call, measured with CUDA events."""
        a, b = C.c_float(0), C.c_float(0)
        cabi.check(self._lib.qw3_last_timing(self._h, C.byref(a), C.byref(b)), "qw3_last_timing")
        return a.value, b.value

    def last_launches(self):
        n = C.c_int64(0)
        cabi.check(self._lib.qw3_last_launches(self._h, C.byref(n)), "qw3_last_launches")
        return n.value

    def kv_upload(self, layer, which, host_f16, upto):
        cabi.check(self._lib.qw3_kv_upload(self._h, layer, which, host_f16.ctypes.data_as(C.c_void_p), upto), "qw3_kv_upload")

    def layer_decode(self, layer, pos, hidden_f16):
        """runOneLayer (Inference.cu:1029-1230) for one token; returns the updated hidden state."""
        import numpy as np
        h = np.ascontiguousarray(hidden_f16).copy()
        cabi.check(self._lib.qw3_layer_decode(self._h, layer, pos, h.ctypes.data_as(C.c_void_p)), "qw3_layer_decode")
        return h

    def stage_hidden(self, stage):
        """Hidden state a stage of this process holds after its last pass (test hook)."""
        import numpy as np
        h = np.empty(self.config.hidden, np.float16)
        cabi.check(self._lib.qw3_stage_hidden(self._h, stage, h.ctypes.data_as(C.c_void_p)), "qw3_stage_hidden")
        return h

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.qw3_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
