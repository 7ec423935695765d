"""Pins the C oracle (oracle/w4a32_oracle.c) to the reference.

Two anchors: the golden vectors under tests/golden/ (made by tests/golden/make_golden.py from the
reference's scalar code compiled in place) and, where that compiled code is present
(oracle/_ref/libkai_ref.so), a direct bit-for-bit comparison on further random shapes.
The reference's own acceptance rule for this path is |ref - act| <= 1e-4
(tests/Arm/KaiLinearTest.hpp:456-463); the oracle is held to exact equality instead.
"""
import hashlib
import os

import numpy as np
import pytest

from oracle_lib import Oracle, load_kai_ref

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "kai_ref_golden.npz"))
RAGGED = sorted({k[:-2] for k in GOLD.files if k.startswith("r_") and k.endswith("_x")})


@pytest.fixture(scope="module")
def orc():
    return Oracle()


def test_reference_fixture_against_golden(orc):
    M, K, N = 1, 1024, 1024
    x = orc.fill_uniform_random(M * K, 4568).reshape(M, K)
    w = orc.fill_uniform_random(N * K, 4572).reshape(N, K)
    assert np.array_equal(x[0, :16], GOLD["fixture_x_head"])
    assert np.array_equal(w[0, :16], GOLD["fixture_w_head"])
    q, s = orc.quant_weights(w)
    assert hashlib.sha256(q.tobytes()).digest() == GOLD["fixture_q_sha256"].tobytes()
    assert hashlib.sha256(s.tobytes()).digest() == GOLD["fixture_s_sha256"].tobytes()
    assert np.array_equal(q[0], GOLD["fixture_q_row0"])
    assert np.array_equal(s[0], GOLD["fixture_s_row0"])
    a = orc.quant_act(x)
    assert np.array_equal(a, GOLD["fixture_a"])
    y = orc.matmul(a, q, s, K)
    assert np.array_equal(y.view(np.uint32), GOLD["fixture_y"].view(np.uint32))
    assert np.max(np.abs(y - GOLD["fixture_y"])) <= 1e-4  # the reference's own tolerance


@pytest.mark.parametrize("name", RAGGED)
def test_ragged_against_golden(orc, name):
    x, w = GOLD[name + "_x"], GOLD[name + "_w"]
    q, s = orc.quant_weights(w)
    assert np.array_equal(q, GOLD[name + "_q"])
    assert np.array_equal(s, GOLD[name + "_s"])
    a = orc.quant_act(x)
    assert np.array_equal(a, GOLD[name + "_a"])
    y = orc.matmul(a, q, s, x.shape[1])
    assert np.array_equal(y.view(np.uint32), GOLD[name + "_y"].view(np.uint32))


def test_bf16_cast_against_golden(orc):
    got = np.array([orc.lib.oracle_cast_bf16_f32(float(v), 0) for v in GOLD["bf16_in"]], np.uint16)
    assert np.array_equal(got, GOLD["bf16_out"])
    for v in GOLD["bf16_out"]:
        f = orc.lib.oracle_cast_f32_bf16(int(v))
        assert np.float32(f).view(np.uint32) == np.uint32(int(v) << 16)


def test_bf16_rne_and_fp16_modes(orc):
    import torch
    vals = torch.tensor([0.0028571, -0.0028571, 1.00390625, 1.01171875, 3.3e-5, 7e-8, 65519.0, 0.1, -2.5e-3],
                        dtype=torch.float32)
    bf = vals.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    hf = vals.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    for v, b, h in zip(vals.tolist(), bf, hf):
        assert orc.lib.oracle_cast_bf16_f32(v, 1) == b
        assert orc.lib.oracle_cast_f16_f32(v) == h
        assert np.float32(orc.lib.oracle_cast_f32_f16(int(h))) == torch.tensor([int(h)], dtype=torch.uint16).view(
            torch.float16).float().item()


def test_nibble_layout_and_quirks(orc):
    # one row, K = 5 (odd, short block): even k -> low nibble, odd k -> high nibble, zero-point 8
    w = np.array([[0.7, -0.35, 0.0, 0.175, -0.7]], np.float32)
    q, s = orc.quant_weights(w)
    # |max| first hit is +0.7 -> scale = 0.7 / -8 (negative); q = round(x / scale)
    scale = np.float32(np.float64(np.float32(0.7)) / -8.0)
    assert s[0, 0] == (scale.view(np.uint32) >> 16)
    qv = [-8, 4, 0, -2, 7]  # +0.7 -> -8 ; -0.7 -> round(8) clamps to 7
    expect = [(qv[0] + 8) | ((qv[1] + 8) << 4), (qv[2] + 8) | ((qv[3] + 8) << 4), (qv[4] + 8)]
    assert q[0].tolist() == expect
    # an all-zero block has scale 0 / -8 = -0.0 (bf16 0x8000) and every nibble equal to the zero point
    q0, s0 = orc.quant_weights(np.zeros((1, 32), np.float32))
    assert s0[0, 0] == 0x8000 and np.all(q0 == 0x88)


def test_act_quant_degenerate_rows(orc):
    x = np.zeros((3, 40), np.float32)
    x[1, :] = 0.25
    x[2, :] = -3.0
    a = orc.quant_act(x)
    hdr = a[:, :8].copy().view(np.float32)[:, 0], a[:, :8].copy().view(np.int32)[:, 1]
    assert hdr[0][0] == 1.0 and hdr[1][0] == -127         # rmin == rmax -> scale 1, zero point 127
    assert np.all(a[0, 8:] == 127)                        # (a_q + a_off) = 0 for every element
    assert np.all(a[1, 8:] == 127) and hdr[1][1] == 128   # all-positive row: zero point -128
    assert np.all(a[2, 8:] == -128) and hdr[1][2] == -127


@pytest.mark.skipif(load_kai_ref() is None, reason="reference build (oracle/_ref/libkai_ref.so) not present")
@pytest.mark.parametrize("m,n,k,seed", [(1, 64, 1536, 1), (4, 37, 1000, 2), (7, 16, 8960, 3), (2, 3, 31, 4),
                                        (16, 24, 1176, 5)])
def test_oracle_equals_compiled_reference(orc, m, n, k, seed):
    ref = load_kai_ref()
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((m, k)) * rng.uniform(0.1, 4.0)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    q, s = orc.quant_weights(w)
    q_r = np.zeros_like(q)
    s_r = np.zeros_like(s)
    ref.kairef_quant_nxk_qs4c32_f32(n, k, 32, w, q_r, s_r)
    assert np.array_equal(q, q_r) and np.array_equal(s, s_r)
    a = orc.quant_act(x)
    a_r = np.zeros_like(a)
    ref.kairef_quant_qa8dx_f32(m, k, x, a_r)
    assert np.array_equal(a, a_r)
    y = orc.matmul(a, q, s, k)
    y_r = np.zeros_like(y)
    ref.kairef_matmul(m, n, k, 32, a_r, q_r, s_r, y_r)
    assert np.array_equal(y.view(np.uint32), y_r.view(np.uint32))


def test_bias_position(orc):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((2, 64)).astype(np.float32)
    w = (rng.standard_normal((6, 64)) * 0.02).astype(np.float32)
    b = rng.standard_normal(6).astype(np.float32)
    q, s = orc.quant_weights(w)
    y0 = orc.linear(x, q, s)
    y1 = orc.linear(x, q, s, bias=b)
    assert np.array_equal(y1, y0 + b[None, :])
