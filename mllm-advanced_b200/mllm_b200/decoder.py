"""ctypes driver of the decoder section of the C ABI (include/mllmb200.h, mllmb200_qwen2_*).

Mirrors how the reference project's model is used: construct from a config
(mllm/Models/ds_qwen2/configuration_ds_qwen2.hpp), load parameters by name, then prefill + greedy
decode (mllm/Models/AutoLLM.hpp:39-65).  torch only holds the device buffers.
"""
import ctypes as C

import numpy as np

from . import binding as B

LINEAR_NAMES = ("q", "k", "v", "o", "gate", "up", "down")


class Qwen2Config(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "inter", "vocab",
                                       "max_ctx")] + [("eps", C.c_float), ("rope_theta", C.c_float)]


# DeepSeek-R1-Distill-Qwen-1.5B / Qwen2-1.5B shapes (configuration_ds_qwen2.hpp defaults)
QWEN2_1P5B = dict(layers=28, hidden=1536, q_heads=12, kv_heads=2, head_dim=128, inter=8960, vocab=151936,
                  max_ctx=1024, eps=1e-6, rope_theta=1000000.0)

DECODE_AUTO, DECODE_GRAPH, DECODE_PERSISTENT = 0, 1, 2
_bound = False


def plan_check(cfg, nctas):
    """Host-only consistency check of the persistent kernel's work plan: (max chunks per CTA and
    layer, max partial-sum slots per row, chunks per layer over all CTAs)."""
    L = _bind()
    a, b, c = C.c_int(), C.c_int(), C.c_int()
    B._check(L.mllmb200_qwen2_plan_check(C.byref(Qwen2Config(**cfg)), nctas, C.byref(a), C.byref(b), C.byref(c)),
             "qwen2_plan_check")
    return a.value, b.value, c.value


def _bind():
    global _bound
    L = B.lib()
    if _bound:
        return L
    vp, ci = C.c_void_p, C.c_int
    L.mllmb200_qwen2_create.argtypes = [C.POINTER(Qwen2Config), C.POINTER(vp)]
    L.mllmb200_qwen2_destroy.argtypes = [vp]
    L.mllmb200_qwen2_destroy.restype = None
    L.mllmb200_qwen2_set_linear.argtypes = [vp, ci, ci, vp, ci, ci, ci, ci]
    L.mllmb200_qwen2_set_linear_tiled.argtypes = [vp, ci, ci, vp]
    L.mllmb200_qwen2_set_norm.argtypes = [vp, ci, ci, vp]
    L.mllmb200_qwen2_set_tables.argtypes = [vp, vp, vp]
    L.mllmb200_qwen2_prefill.argtypes = [vp, vp, ci]
    L.mllmb200_qwen2_decode.argtypes = [vp, ci]
    L.mllmb200_qwen2_decode_ex.argtypes = [vp, ci, ci]
    L.mllmb200_qwen2_plan_check.argtypes = [C.POINTER(Qwen2Config), ci, C.POINTER(ci), C.POINTER(ci), C.POINTER(ci)]
    L.mllmb200_qwen2_read.argtypes = [vp, ci, ci, vp, vp, vp]
    L.mllmb200_qwen2_set_profiling.argtypes = [vp, ci]
    L.mllmb200_qwen2_phase_cycles.argtypes = [vp, vp, ci, C.POINTER(ci), C.POINTER(ci)]
    L.mllmb200_qwen2_stream.argtypes = [vp]
    L.mllmb200_qwen2_stream.restype = vp
    L.mllmb200_qwen2_batch_create.argtypes = [vp, ci, C.POINTER(vp)]
    L.mllmb200_qwen2_batch_destroy.argtypes = [vp]
    L.mllmb200_qwen2_batch_destroy.restype = None
    L.mllmb200_qwen2_batch_set_policy.argtypes = [vp, ci]
    L.mllmb200_qwen2_batch_prefill.argtypes = [vp, ci, vp, vp, ci]
    L.mllmb200_qwen2_batch_decode.argtypes = [vp, ci]
    L.mllmb200_qwen2_batch_read.argtypes = [vp, ci, ci, ci, vp, vp, vp]
    _bound = True
    return L


class Qwen2Decoder:
    def __init__(self, cfg, device="cuda"):
        import torch
        self.cfg = dict(cfg)
        self.device = torch.device(device)
        self._L = _bind()
        self._h = C.c_void_p()
        self._keep = []
        with torch.cuda.device(self.device):
            B._check(self._L.mllmb200_qwen2_create(C.byref(Qwen2Config(**self.cfg)), C.byref(self._h)), "qwen2_create")
        self.prompt_len = 0

    def close(self):
        if self._h:
            self._L.mllmb200_qwen2_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_linear(self, layer, name, blob):
        """blob: host pre-pack blob (numpy uint8) of the [N, K] weight (+ bias)."""
        import torch
        n, k, sm, hb = B.blob_info(blob)
        dev = torch.from_numpy(blob).to(self.device)
        B._check(self._L.mllmb200_qwen2_set_linear(self._h, layer, LINEAR_NAMES.index(name), dev.data_ptr(), n, k, sm, hb),
                 f"qwen2_set_linear({layer},{name})")

    def set_linear_tiled(self, layer, name, weights):
        """weights: binding.W4A32Weights of the whole matrix (borrowed; kept alive by this object)."""
        self._keep_w = getattr(self, "_keep_w", []) + [weights]
        B._check(self._L.mllmb200_qwen2_set_linear_tiled(self._h, layer, LINEAR_NAMES.index(name),
                                                         weights.tiled.data_ptr()), "qwen2_set_linear_tiled")

    def set_norm(self, kind, layer, w):
        import torch
        dev = torch.from_numpy(np.ascontiguousarray(w, np.float32)).to(self.device)
        B._check(self._L.mllmb200_qwen2_set_norm(self._h, kind, layer, dev.data_ptr()), "qwen2_set_norm")

    def set_tables(self, embedding, lm_head_f16):
        """torch tensors on the device: fp32 [V,H] and fp16 [V,H]; kept alive by this object."""
        self._keep = [embedding, lm_head_f16]
        B._check(self._L.mllmb200_qwen2_set_tables(self._h, embedding.data_ptr(), lm_head_f16.data_ptr()),
                 "qwen2_set_tables")

    def prefill(self, tokens):
        import torch
        t = torch.as_tensor(np.asarray(tokens, np.int32)).to(self.device)
        self._keep_tokens = t
        self.prompt_len = int(t.numel())
        B._check(self._L.mllmb200_qwen2_prefill(self._h, t.data_ptr(), self.prompt_len), "qwen2_prefill")

    def prefill_device(self, tokens_dev):
        self._keep_tokens = tokens_dev
        self.prompt_len = int(tokens_dev.numel())
        B._check(self._L.mllmb200_qwen2_prefill(self._h, tokens_dev.data_ptr(), self.prompt_len), "qwen2_prefill")

    def decode(self, steps, mode=0):
        """mode: DECODE_AUTO, DECODE_GRAPH (one graph replay per step) or DECODE_PERSISTENT (one launch)."""
        B._check(self._L.mllmb200_qwen2_decode_ex(self._h, steps, mode), "qwen2_decode")

    def read(self, first, count, want_logits=False):
        toks = np.zeros(max(count, 1), np.int32)
        pos = C.c_int(0)
        logits = np.zeros(self.cfg["vocab"], np.float32) if want_logits else None
        B._check(self._L.mllmb200_qwen2_read(self._h, first, count, toks.ctypes.data, C.byref(pos),
                                             logits.ctypes.data if want_logits else None), "qwen2_read")
        return toks[:count], pos.value, logits

    def generated(self, steps):
        """Tokens sampled after the prompt and after each of `steps` decode steps."""
        return self.read(self.prompt_len - 1, steps + 1)[0]

    def set_profiling(self, on):
        B._check(self._L.mllmb200_qwen2_set_profiling(self._h, int(bool(on))), "qwen2_set_profiling")

    def phase_cycles(self):
        """[nctas, stamps] clock cycles per phase of the last persistent launch."""
        n, k = C.c_int(), C.c_int()
        B._check(self._L.mllmb200_qwen2_phase_cycles(self._h, None, 0, C.byref(n), C.byref(k)), "qwen2_phase_cycles")
        out = np.zeros((n.value, k.value), np.int64)
        B._check(self._L.mllmb200_qwen2_phase_cycles(self._h, out.ctypes.data, out.size, C.byref(n), C.byref(k)),
                 "qwen2_phase_cycles")
        return out

    def stream(self):
        import torch
        return torch.cuda.ExternalStream(self._L.mllmb200_qwen2_stream(self._h), device=self.device)


class Qwen2BatchDecoder:
    """`batch` sequences decoding together on the weights of a Qwen2Decoder (mllmb200_qwen2_batch_*): every
    sequence has its own KV cache and position; sequence b yields what the batch-1 decoder yields on it alone."""

    def __init__(self, decoder, batch):
        import torch
        self.dec = decoder
        self.batch = int(batch)
        self._L = _bind()
        self._h = C.c_void_p()
        self._keep = []
        self.prompt_len = [0] * self.batch
        with torch.cuda.device(decoder.device):
            B._check(self._L.mllmb200_qwen2_batch_create(decoder._h, self.batch, C.byref(self._h)), "qwen2_batch_create")

    def close(self):
        if self._h:
            self._L.mllmb200_qwen2_batch_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_policy(self, policy):
        B._check(self._L.mllmb200_qwen2_batch_set_policy(self._h, policy), "qwen2_batch_set_policy")

    def prefill(self, seq, tokens=None, embeds=None):
        """tokens: int sequence, or embeds: torch fp32 [n, hidden] on the device (rows that already are embeddings)."""
        import torch
        if tokens is not None:
            t = tokens if isinstance(tokens, torch.Tensor) else torch.as_tensor(np.asarray(tokens, np.int32)).to(self.dec.device)
            self._keep.append(t)
            n = int(t.numel())
            B._check(self._L.mllmb200_qwen2_batch_prefill(self._h, seq, t.data_ptr(), None, n), "qwen2_batch_prefill")
        else:
            assert embeds.is_cuda and embeds.dtype == torch.float32 and embeds.is_contiguous()
            self._keep.append(embeds)
            n = int(embeds.shape[0])
            B._check(self._L.mllmb200_qwen2_batch_prefill(self._h, seq, None, embeds.data_ptr(), n), "qwen2_batch_prefill")
        self.prompt_len[seq] = n

    def decode(self, steps):
        B._check(self._L.mllmb200_qwen2_batch_decode(self._h, steps), "qwen2_batch_decode")

    def read(self, seq, first, count, want_logits=False):
        toks = np.zeros(max(count, 1), np.int32)
        pos = C.c_int(0)
        logits = np.zeros(self.dec.cfg["vocab"], np.float32) if want_logits else None
        B._check(self._L.mllmb200_qwen2_batch_read(self._h, seq, first, count, toks.ctypes.data, C.byref(pos),
                                                   logits.ctypes.data if want_logits else None), "qwen2_batch_read")
        return toks[:count], pos.value, logits

    def generated(self, seq, steps):
        """Tokens sampled after the prompt of `seq` and after each of `steps` decode steps."""
        return self.read(seq, self.prompt_len[seq] - 1, steps + 1)[0]
