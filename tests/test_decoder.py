"""Decoder tests: the CUDA Qwen2-architecture decoder (C ABI mllmb200_qwen2_*) against the numpy
restatement oracle/qwen2_oracle.py whose linears are the W4A32 C oracle.

Bars: logits max|diff| <= 5e-3 * rms(logits) (fp32 throughout), and the greedy tokens identical - a
differing token is accepted only where the oracle's own margin between the two candidates is below
the logit bar.  The int8 activation quantization in front of every linear can turn a last-bit
difference of its input into a whole quantization step (worst: a row's zero point moves by one), so
a case can be ill-conditioned: the oracle is therefore also run on an embedding table scaled by
(1 +- 2e-7), and where ITS logits move by more than the bar, the bar of that case is 3x that move."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
from qwen2_oracle import Qwen2Oracle, rmsnorm, rope, rope_tables  # noqa: E402
from oracle_lib import Oracle  # noqa: E402

LOGIT_TOL = 5e-3
STEPWISE_TOL = 2e-2  # oracle prompt-at-once vs token-by-token (different summation orders in numpy)

SMALL = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, inter=512, vocab=1000, max_ctx=96, eps=1e-6,
             rope_theta=10000.0)
WIDE = dict(layers=3, hidden=512, q_heads=4, kv_heads=2, head_dim=128, inter=1184, vocab=3001, max_ctx=128, eps=1e-6,
            rope_theta=1000000.0)
# BASELINE config 2 at full size: every width and all 28 layers of the 1.5B architecture
FULL = dict(layers=28, hidden=1536, q_heads=12, kv_heads=2, head_dim=128, inter=8960, vocab=151936, max_ctx=64, eps=1e-6,
            rope_theta=1000000.0)
_CASE_CACHE = {}  # (config id, seed, prompt length, steps) -> model and oracle results, shared by the two decode modes


def make_model(cfg, seed):
    """Random-init weights: returns (oracle weights dict, list of (layer, name, w, bias))."""
    rng = np.random.default_rng(seed)
    H, QD, KD, I, V = (cfg["hidden"], cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"], cfg["inter"],
                       cfg["vocab"])
    shapes = dict(q=(QD, H), k=(KD, H), v=(KD, H), o=(H, QD), gate=(I, H), up=(I, H), down=(H, I))
    raw = []
    w = {"embedding": rng.standard_normal((V, H)).astype(np.float32),
         "lm_head": (rng.standard_normal((V, H)) * 0.05).astype(np.float16).astype(np.float32),
         "final_norm": (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)}
    for l in range(cfg["layers"]):
        w[f"ln1.{l}"] = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        w[f"ln2.{l}"] = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        for name, (n, k) in shapes.items():
            wt = (rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32)
            b = (0.1 * rng.standard_normal(n)).astype(np.float32) if name in ("q", "k", "v") else None
            raw.append((l, name, wt, b))
    return w, raw


def bind_oracle_linears(w, raw, orc):
    for l, name, wt, b in raw:
        q, s = orc.quant_weights(wt)
        w[f"{name}.{l}"] = (lambda x, q=q, s=s, b=b: orc.linear(x, q, s, b))
    return w


# ------------------------------------------------------------------ CPU: the oracle itself
def test_oracle_prefill_equals_stepwise():
    """Feeding a prompt at once and token by token must agree (KV cache, mask, positions)."""
    orc = Oracle()
    w, raw = make_model(SMALL, 1)
    bind_oracle_linears(w, raw, orc)
    m = Qwen2Oracle(SMALL, w)
    prompt = [3, 17, 999, 0, 5, 42]
    a = m.forward(prompt)
    m.reset()
    for t in prompt:
        b = m.forward([t])
    rms = float(np.sqrt(np.mean(a.astype(np.float64) ** 2)))
    assert np.max(np.abs(a - b)) <= STEPWISE_TOL * rms


def test_oracle_operator_identities():
    x = np.random.default_rng(0).standard_normal((3, 64)).astype(np.float32)
    y = rmsnorm(x, np.ones(64, np.float32), 0.0)
    assert np.allclose((y * y).mean(-1), 1.0, atol=1e-5)
    sin_t, cos_t = rope_tables(16, 64, 10000.0)
    q = x.reshape(3, 1, 64)
    r = rope(q, np.array([0, 5, 9]), sin_t, cos_t)
    assert np.array_equal(r[0], q[0])                                    # position 0 is the identity
    assert np.allclose((r * r).sum(-1), (q * q).sum(-1), rtol=1e-5)        # rotations keep the norm
    # the score of a rotated pair depends on the distance only
    a = rope(q[:1], np.array([3]), sin_t, cos_t)[0, 0] @ rope(q[1:2], np.array([7]), sin_t, cos_t)[0, 0]
    b = rope(q[:1], np.array([8]), sin_t, cos_t)[0, 0] @ rope(q[1:2], np.array([12]), sin_t, cos_t)[0, 0]
    assert abs(a - b) <= 1e-3 * (abs(a) + 1.0)


def test_config_struct_matches_header():
    import ctypes as C
    from mllm_b200.decoder import Qwen2Config
    assert C.sizeof(Qwen2Config) == 40
    hdr = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "mllmb200.h")).read()
    assert "int layers, hidden, q_heads, kv_heads, head_dim, inter, vocab, max_ctx;" in hdr
    assert "float eps, rope_theta;" in hdr


@pytest.mark.parametrize("nctas", [1, 7, 132, 148, 160])
def test_persistent_plan_covers_every_cell_once(nctas):
    """The static work plan of the persistent decode kernel (host code): the library's own checker
    walks every chunk of every CTA; here also the chunk totals against the cell counts."""
    import mllm_b200 as mb
    for cfg in (SMALL, WIDE, dict(mb.QWEN2_1P5B)):
        max_chunks, max_slots, total = mb.plan_check(cfg, nctas)
        H, QD, KD, I = cfg["hidden"], cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"], cfg["inter"]
        cells = ((QD + 2 * KD) * H + H * QD + 2 * I * H + H * I) // (32 * 32)
        assert 1 <= max_slots <= 8 and max_chunks >= 1
        assert cells / 16 <= total <= cells  # chunks hold 1..16 cells
    with pytest.raises(mb.MllmB200Error):
        mb.plan_check(dict(SMALL, hidden=250), 148)


# ------------------------------------------------------------------ GPU
def _gpu_decoder(cfg, w, raw):
    import torch
    import mllm_b200 as mb
    dec = mb.Qwen2Decoder(cfg)
    for l, name, wt, b in raw:
        dec.set_linear(l, name, mb.quant_prepack(wt, b))
    for l in range(cfg["layers"]):
        dec.set_norm(0, l, w[f"ln1.{l}"])
        dec.set_norm(1, l, w[f"ln2.{l}"])
    dec.set_norm(2, 0, w["final_norm"])
    dec.set_tables(torch.from_numpy(w["embedding"]).cuda(), torch.from_numpy(w["lm_head"].astype(np.float16)).cuda())
    return dec


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [1, 2], ids=["graph", "persistent"])
@pytest.mark.parametrize("cfg,seed,prompt_len,steps", [(SMALL, 11, 3, 20), (SMALL, 12, 9, 12), (SMALL, 13, 40, 24),
                                                       (WIDE, 14, 1, 10), (WIDE, 15, 33, 16), (FULL, 16, 4, 4)],
                         ids=["small-3", "small-9", "small-40", "wide-1", "wide-33", "full-1p5b-4"])
def test_decoder_matches_oracle(cfg, seed, prompt_len, steps, mode):
    import torch
    import mllm_b200 as mb
    assert torch.cuda.is_available()
    key = (id(cfg), seed, prompt_len, steps)
    if key not in _CASE_CACHE:
        _CASE_CACHE.clear()  # one case at a time: the full-size model is several GB
        orc = Oracle()
        w, raw = make_model(cfg, seed)
        bind_oracle_linears(w, raw, orc)
        prompt = np.random.default_rng(seed + 100).integers(0, cfg["vocab"], prompt_len).tolist()
        ref_toks, ref_logits = Qwen2Oracle(cfg, w).generate(prompt, steps)
        # conditioning of the case: how far the oracle's own logits move under a last-bit input change
        bars = np.full(steps + 1, LOGIT_TOL)
        for eps in (2e-7, -2e-7):
            w2 = dict(w, embedding=(w["embedding"] * np.float32(1.0 + eps)).astype(np.float32))
            ptoks, plogits = Qwen2Oracle(cfg, w2).generate(prompt, steps)
            for i in range(steps + 1):
                rms = float(np.sqrt(np.mean(ref_logits[i].astype(np.float64) ** 2)))
                bars[i] = max(bars[i], 3.0 * float(np.max(np.abs(plogits[i] - ref_logits[i]))) / rms)
                if ptoks[i] != ref_toks[i]:
                    bars[i + 1:] = np.inf  # the perturbed oracle itself left the sequence: nothing to compare after
                    break
        bars = np.maximum.accumulate(bars)  # a moved cache entry stays in the cache
        _CASE_CACHE[key] = (w, raw, prompt, ref_toks, ref_logits, bars)
    w, raw, prompt, ref_toks, ref_logits, bars = _CASE_CACHE[key]

    def rel_err(got, i):
        rms = float(np.sqrt(np.mean(ref_logits[i].astype(np.float64) ** 2)))
        return float(np.max(np.abs(got - ref_logits[i]))) / rms

    dec = _gpu_decoder(cfg, w, raw)
    dec.prefill(prompt)
    toks0, pos0, logits0 = dec.read(prompt_len - 1, 1, want_logits=True)
    assert pos0 == prompt_len
    errs = [rel_err(logits0, 0)]
    assert errs[0] <= bars[0], f"prefill logits: {errs[0]:.3e} > {bars[0]:.3e}"
    # step by step first (logits after every step), then the same again in one call
    got = [int(toks0[0])]
    for i in range(steps):
        if got[-1] != ref_toks[i]:
            break
        dec.decode(1, mode)
        t, pos, lg = dec.read(prompt_len + i, 1, want_logits=True)
        assert pos == prompt_len + i + 1
        errs.append(rel_err(lg, i + 1))
        assert errs[-1] <= bars[i + 1], f"logits of step {i}: {errs[-1]:.3e} > {bars[i + 1]:.3e}"
        got.append(int(t[0]))
    print(f"decoder parity mode={mode} hidden={cfg['hidden']} prompt={prompt_len}: max rel logit err {max(errs):.3e}, "
          f"bar {bars[0]:.1e}..{bars[len(errs) - 1]:.1e}, {len(got)} tokens")
    for i, (a, b) in enumerate(zip(got, ref_toks)):
        if a != b:
            margin = abs(float(ref_logits[i][a]) - float(ref_logits[i][b]))
            rms = float(np.sqrt(np.mean(ref_logits[i].astype(np.float64) ** 2)))
            assert margin <= bars[i] * rms, f"token {i}: {a} vs {b}, oracle margin {margin:.3e}"
            break
    else:
        assert len(got) == steps + 1
    # a fresh prefill + all steps in one call (graph replays back to back) gives the same tokens
    dec.prefill(prompt)
    dec.decode(len(got) - 1, mode)
    again = dec.generated(len(got) - 1)
    assert again.tolist() == got
    mb.check_device_status()
    dec.close()


@pytest.mark.gpu
def test_decoder_rejects_bad_arguments():
    import mllm_b200 as mb
    with pytest.raises(mb.MllmB200Error):
        mb.Qwen2Decoder(dict(SMALL, head_dim=48))
    dec = mb.Qwen2Decoder(SMALL)
    with pytest.raises(mb.MllmB200Error):
        dec.decode(1)  # no weights yet
    w = np.zeros((64, 64), np.float32)
    with pytest.raises(mb.MllmB200Error):
        dec.set_linear(0, "q", mb.quant_prepack(w))  # wrong shape for this config
    dec.close()


@pytest.mark.gpu
@pytest.mark.parametrize("prompt_len", [64, 400])
def test_full_width_decode_agrees_with_prefill(prompt_len):
    """Size-independent property at the full Qwen2-1.5B widths (4 layers): tokens produced by decode
    steps (GEMV kernels, fused quantizing producers, graph replay) and the token a from-scratch
    prefill of prompt + those tokens samples (tcgen05 kernels, separate quantization) come from the
    same function, so the logits agree within the case bar and the sampled token is the same."""
    import torch
    import mllm_b200 as mb
    import bench
    gen = torch.Generator(device="cuda").manual_seed(5)
    cfg = dict(mb.QWEN2_1P5B, layers=4, max_ctx=512)  # (400 positions: 13 key blocks per attention tile at the end of the prompt)
    layers = [[bench.make_random_weights(mb, torch, n, k, hb, gen) for _, k, n, hb in bench.LINEARS] for _ in range(4)]
    dec = mb.Qwen2Decoder(cfg)
    for l, lw in enumerate(layers):
        for (name, _, _, _), wt in zip(bench.LINEARS, lw):
            dec.set_linear_tiled(l, name, wt)
        for kind in (0, 1):
            dec.set_norm(kind, l, np.ones(cfg["hidden"], np.float32))
    dec.set_norm(2, 0, np.ones(cfg["hidden"], np.float32))
    emb = torch.randn((cfg["vocab"], cfg["hidden"]), device="cuda", generator=gen)
    head = (torch.randn((cfg["vocab"], cfg["hidden"]), device="cuda", generator=gen) * 0.02).to(torch.float16)
    dec.set_tables(emb, head)
    prompt = np.random.default_rng(3).integers(0, cfg["vocab"], prompt_len).tolist()
    steps = 8
    dec.prefill(prompt)
    dec.decode(steps)
    toks = dec.generated(steps).tolist()
    _, pos, lg_decode = dec.read(0, 0, want_logits=True)
    assert pos == prompt_len + steps
    dec.prefill(prompt + toks[:steps])
    t2, pos2, lg_prefill = dec.read(prompt_len + steps - 1, 1, want_logits=True)
    assert pos2 == prompt_len + steps
    rms = float(np.sqrt(np.mean(lg_prefill.astype(np.float64) ** 2)))
    err = float(np.max(np.abs(lg_decode - lg_prefill))) / rms
    print(f"full-width decode vs prefill: rel logit err {err:.3e}")
    assert err <= 2e-2
    assert int(t2[0]) == toks[steps] or abs(float(lg_prefill[int(t2[0])] - lg_prefill[toks[steps]])) <= 2e-2 * rms
    mb.check_device_status()
    dec.close()
