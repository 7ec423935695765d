"""CPU restatement (numpy, fp32) of the reference project's Qwen2-architecture decoder forward.

TEST INFRASTRUCTURE ONLY: the checker for the CUDA decoder; nothing shipped imports it.

Follows, in the reference project:
  mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:47-54    MLP  down(silu(gate(x)) * up(x))
  mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:106-155  attention: q/k/v linears, RoPE on q and k, KV cache,
                                                      q.k^T * 1/sqrt(D), causal mask, softmax, .v, o linear
  mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:175-183  decoder layer (pre-norm, two residuals)
  mllm/Models/ds_qwen2/modeling_ds_qwen2.hpp:202-215  embedding, layers, final norm, lm_head product
  mllm/Backends/Arm/Ops/RMSNormOp.cpp:20-77           y = x * w / sqrt(mean(x^2) + eps)
  mllm/Backends/Arm/Kernels/rope.cpp:20-87            half-split rotation, theta = pos * base^(-2d/D)
  mllm/Models/AutoLLM.hpp:39-105                      greedy loop, argmax of the last row
The seven linears are passed in as callables (the tests bind them to the W4A32 C oracle), so this
file restates only the operators around them.  Parity of those operators is "unpinned": the
reference's Arm kernels for them (NEON exp/sigmoid approximations) do not build on this host, so
they are restated from their definitions with libm-grade exp; the tests state the tolerance.
"""
import numpy as np

F = np.float32


def rmsnorm(x, w, eps):
    x = x.astype(F)
    ms = (x * x).sum(-1, keepdims=True, dtype=F) / F(x.shape[-1])
    return (x * (w.astype(F) * (F(1.0) / np.sqrt(ms + F(eps), dtype=F)))).astype(F)


def rope_tables(max_pos, head_dim, base):
    half = head_dim // 2
    d = np.arange(half, dtype=F)
    inv = (F(1.0) / np.power(F(base), F(2.0) * d / F(head_dim), dtype=F)).astype(F)
    theta = (np.arange(max_pos, dtype=F)[:, None] * inv[None, :]).astype(F)
    return np.sin(theta, dtype=F), np.cos(theta, dtype=F)


def rope(x, pos, sin_t, cos_t):
    """x: [S, heads, D]; pos: [S] absolute positions."""
    half = x.shape[-1] // 2
    sn, cs = sin_t[pos][:, None, :], cos_t[pos][:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return np.concatenate([x0 * cs - x1 * sn, x0 * sn + x1 * cs], -1).astype(F)


def silu(x):
    x = x.astype(F)
    return (x / (F(1.0) + np.exp(-x, dtype=F))).astype(F)


class Qwen2Oracle:
    """cfg: dict(layers, hidden, q_heads, kv_heads, head_dim, inter, vocab, max_ctx, eps, rope_theta).
    weights: dict with 'embedding' [V,H] fp32, 'lm_head' [V,H] (already rounded to fp16 values),
    'final_norm', and per layer l: 'ln1.l', 'ln2.l' and callables 'q.l','k.l','v.l','o.l','gate.l',
    'up.l','down.l' mapping fp32 [M,K] -> fp32 [M,N]."""

    def __init__(self, cfg, weights):
        self.c, self.w = cfg, weights
        self.sin_t, self.cos_t = rope_tables(cfg["max_ctx"], cfg["head_dim"], cfg["rope_theta"])
        self.reset()

    def reset(self):
        c = self.c
        self.kc = [np.zeros((0, c["kv_heads"], c["head_dim"]), F) for _ in range(c["layers"])]
        self.vc = [np.zeros((0, c["kv_heads"], c["head_dim"]), F) for _ in range(c["layers"])]
        self.pos = 0

    def forward(self, tokens):
        """Feeds `tokens` at positions pos..pos+S-1; returns the logits of the last row."""
        c, w = self.c, self.w
        S = len(tokens)
        D, QH, KH = c["head_dim"], c["q_heads"], c["kv_heads"]
        pos = np.arange(self.pos, self.pos + S)
        h = w["embedding"][np.asarray(tokens)].astype(F)
        for l in range(c["layers"]):
            x = rmsnorm(h, w[f"ln1.{l}"], c["eps"])
            q = w[f"q.{l}"](x).reshape(S, QH, D)
            k = w[f"k.{l}"](x).reshape(S, KH, D)
            v = w[f"v.{l}"](x).reshape(S, KH, D)
            q = rope(q, pos, self.sin_t, self.cos_t)
            k = rope(k, pos, self.sin_t, self.cos_t)
            self.kc[l] = np.concatenate([self.kc[l], k], 0)
            self.vc[l] = np.concatenate([self.vc[l], v], 0)
            K, V = self.kc[l], self.vc[l]
            out = np.zeros((S, QH, D), F)
            scale = F(1.0) / np.sqrt(F(D))
            for hq in range(QH):
                hk = hq // (QH // KH)
                sc = (q[:, hq, :] @ K[:, hk, :].T).astype(F) * scale       # [S, ctx]
                ctx = np.arange(K.shape[0])[None, :]
                sc = np.where(ctx <= pos[:, None], sc, F(-np.inf))
                sc = np.exp(sc - sc.max(-1, keepdims=True), dtype=F)
                p = (sc / sc.sum(-1, keepdims=True, dtype=F)).astype(F)
                out[:, hq, :] = p @ V[:, hk, :]
            a = w[f"o.{l}"](out.reshape(S, QH * D))
            h = (a + h).astype(F)
            x = rmsnorm(h, w[f"ln2.{l}"], c["eps"])
            m = w[f"down.{l}"]((silu(w[f"gate.{l}"](x)) * w[f"up.{l}"](x)).astype(F))
            h = (m + h).astype(F)
        self.pos += S
        x = rmsnorm(h[-1:], w["final_norm"], c["eps"])
        return (x @ w["lm_head"].astype(F).T).astype(F)[0]

    def generate(self, prompt, steps):
        """Greedy: returns (tokens sampled after the prompt and after each step, list of logits)."""
        self.reset()
        logits = [self.forward(list(prompt))]
        toks = [int(np.argmax(logits[-1]))]
        for _ in range(steps):
            logits.append(self.forward([toks[-1]]))
            toks.append(int(np.argmax(logits[-1])))
        return toks, logits
