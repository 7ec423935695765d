"""Generates tests/golden/kai_ref_golden.npz from the reference's own scalar code.

Run in a container that has the reference tree (it builds oracle/_ref/libkai_ref.so from
tests/Arm/KaiLinearTest.hpp where it lies):

    make -C oracle && python tests/golden/make_golden.py

Cases:
  fixture : the reference's only test of this path, M=1 K=N=1024 bl=32, inputs from glibc
            srand(4568) / srand(4572) (tests/Arm/KaiLinearTest.hpp:387-405).  Stored: the full
            fp32 output, the quantized activation row, and SHA-256 of the nibbles and scales.
  ragged  : small shapes with a short last block, an odd K, negative / zero scales and a
            constant row; inputs, nibbles, scales, quantized activations and outputs stored whole.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_lib import load_kai_ref  # noqa: E402


def run_ref(ref, x, w):
    m, k = x.shape
    n = w.shape[0]
    q = np.zeros((n, (k + 1) // 2), np.uint8)
    s = np.zeros((n, (k + 31) // 32), np.uint16)
    ref.kairef_quant_nxk_qs4c32_f32(n, k, 32, w, q, s)
    a = np.zeros((m, k + 8), np.int8)
    ref.kairef_quant_qa8dx_f32(m, k, x, a)
    y = np.zeros((m, n), np.float32)
    ref.kairef_matmul(m, n, k, 32, a, q, s, y)
    return q, s, a, y


def ragged_inputs():
    cases = {}
    rng = np.random.default_rng(20240607)
    for name, (m, n, k) in {"r_m3_n5_k70": (3, 5, 70), "r_m2_n9_k71": (2, 9, 71), "r_m1_n4_k32": (1, 4, 32),
                            "r_m5_n7_k96": (5, 7, 96), "r_m4_n33_k257": (4, 33, 257)}.items():
        x = rng.standard_normal((m, k)).astype(np.float32)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        w[0, :32] = 0.0                      # zero scale block
        w[1 % n, 0] = 0.5                    # positive max -> negative scale
        w[2 % n, 1] = -0.5                   # negative max -> positive scale
        if m > 1:
            x[1, :] = 0.25                   # constant positive row (rmin = 0)
        if m > 2:
            x[2, :] = 0.0                    # all-zero row (rmin == rmax -> scale 1)
        if m > 3:
            x[3, :] = -np.abs(x[3, :])       # all-negative row (rmax = 0)
        cases[name] = (x, w)
    return cases


def main():
    ref = load_kai_ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libkai_ref.so is missing: run `make -C oracle` where the reference tree exists")
    out = {}
    M, K, N = 1, 1024, 1024
    x = np.empty((M, K), np.float32)
    w = np.empty((N, K), np.float32)
    ref.kairef_fill_uniform_random(M, K, x, 4568)
    ref.kairef_fill_uniform_random(N, K, w, 4572)
    q, s, a, y = run_ref(ref, x, w)
    out["fixture_x_head"] = x[0, :16].copy()
    out["fixture_w_head"] = w[0, :16].copy()
    out["fixture_y"] = y
    out["fixture_a"] = a
    out["fixture_q_sha256"] = np.frombuffer(hashlib.sha256(q.tobytes()).digest(), np.uint8)
    out["fixture_s_sha256"] = np.frombuffer(hashlib.sha256(s.tobytes()).digest(), np.uint8)
    out["fixture_q_row0"] = q[0].copy()
    out["fixture_s_row0"] = s[0].copy()
    for name, (x, w) in ragged_inputs().items():
        q, s, a, y = run_ref(ref, x, w)
        out[name + "_x"] = x
        out[name + "_w"] = w
        out[name + "_q"] = q
        out[name + "_s"] = s
        out[name + "_a"] = a
        out[name + "_y"] = y
    # bf16 cast samples
    vals = np.array([0.0, -0.0, 1.0, -1.0, 0.0028571, -0.0028571, 3.1415927, 1e-30, -65504.0, 1.00390625, 1.0078125],
                    np.float32)
    out["bf16_in"] = vals
    out["bf16_out"] = np.array([ref.kairef_cast_bf16_f32(float(v)) for v in vals], np.uint16)
    path = os.path.join(HERE, "kai_ref_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
