"""CPU-side checks: the C ABI library loads and exports every declared symbol, the host
quantize/pre-pack entry points are bit-identical to the oracle, and argument errors come back
as status codes.  No compute call touches a GPU here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import mllm_b200 as mb
from oracle_lib import Oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "mllmb200.h")).read()
    names = set(re.findall(r"MLLMB200_API\s+[\w\s\*]+?\b(mllmb200_\w+)\s*\(", hdr))
    assert len(names) >= 15
    L = C.CDLL(mb.lib_path())
    for n in sorted(names):
        assert hasattr(L, n), f"{n} declared in include/mllmb200.h but not exported"


def test_status_strings():
    assert mb.status_str(0) == "ok"
    for s in range(1, 7):
        assert mb.status_str(s) not in ("ok", "unknown status")
    assert mb.status_str(99) == "unknown status"


@pytest.mark.parametrize("n,k,mode", [(64, 1536, 0), (5, 70, 0), (9, 71, 1), (33, 257, 2), (7, 32, 0), (256, 1176, 0)])
def test_quant_prepack_bit_exact_vs_oracle(n, k, mode):
    rng = np.random.default_rng(n * 1000 + k)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    w[0, : min(32, k)] = 0.0
    bias = rng.standard_normal(n).astype(np.float32)
    blob = mb.quant_prepack(w, bias, mode)
    assert mb.blob_info(blob) == (n, k, mode, 1)
    nib, sc, b = mb.blob_sections(blob)
    q, s = Oracle().quant_weights(w, mode)
    assert np.array_equal(nib, q)
    assert np.array_equal(sc, s)
    assert np.array_equal(b, bias)


def test_quant_prepack_reference_fixture_golden():
    import hashlib
    gold = np.load(os.path.join(ROOT, "tests", "golden", "kai_ref_golden.npz"))
    o = Oracle()
    w = o.fill_uniform_random(1024 * 1024, 4572).reshape(1024, 1024)
    nib, sc, b = mb.blob_sections(mb.quant_prepack(w))
    assert b is None
    assert hashlib.sha256(np.ascontiguousarray(nib).tobytes()).digest() == gold["fixture_q_sha256"].tobytes()
    assert hashlib.sha256(np.ascontiguousarray(sc).tobytes()).digest() == gold["fixture_s_sha256"].tobytes()


def test_prepack_from_quantized_roundtrip():
    rng = np.random.default_rng(3)
    n, k = 40, 96
    q = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    s = rng.integers(0, 65536, (n, k // 32), dtype=np.uint16)
    blob = mb.prepack_from_quantized(q, s, n, k, None, mb.SCALE_FP16)
    nib, sc, b = mb.blob_sections(blob)
    assert np.array_equal(nib, q) and np.array_equal(sc, s) and b is None
    assert mb.blob_info(blob) == (n, k, 2, 0)


def test_error_statuses():
    L = mb.lib()
    out = C.c_size_t()
    assert L.mllmb200_w4a32_prepack_size(0, 32, 0, C.byref(out)) == 1
    assert L.mllmb200_w4a32_prepack_size(8, -1, 0, C.byref(out)) == 1
    assert L.mllmb200_w4a32_prepack_size(8, 32, 0, None) == 1
    assert L.mllmb200_w4a32_prepack_size(1 << 20, 1 << 14, 0, C.byref(out)) == 2  # >= 2 GiB blob
    assert L.mllmb200_w4a32_tiled_size(8, 0, C.byref(out)) == 1
    assert L.mllmb200_w4a32_workspace_size(0, 32, C.byref(out)) == 1
    bad = np.zeros(128, np.uint8)
    assert L.mllmb200_w4a32_blob_info(bad.ctypes.data, bad.size, None, None, None, None) == 5
    good = mb.quant_prepack(np.ones((4, 32), np.float32))
    assert L.mllmb200_w4a32_blob_info(good.ctypes.data, good.size - 16, None, None, None, None) == 5  # truncated
    good[8] ^= 0xFF  # corrupt N
    assert L.mllmb200_w4a32_blob_info(good.ctypes.data, good.size, None, None, None, None) == 5
    w = np.ones((4, 32), np.float32)
    blob = np.zeros(1024, np.uint8)
    assert L.mllmb200_w4a32_quant_prepack(None, None, 4, 32, 0, blob.ctypes.data) == 1
    assert L.mllmb200_w4a32_quant_prepack(w.ctypes.data, None, 4, 32, 7, blob.ctypes.data) == 1
    # device entry points reject bad arguments before touching the GPU
    assert L.mllmb200_w4a32_linear_forward(None, None, None, None, 1, 32, 32, 32, 32, None) == 1
    assert L.mllmb200_w4a32_repack_device(None, 4, 32, 0, 0, 0, 4, None, None) == 1


def test_sizes():
    # blob: 64-byte header + nibbles + scales (+ bias), sections 16-byte aligned
    assert mb.prepack_size(8960, 1536, 0) == 64 + 8960 * 768 + 8960 * 96
    assert mb.prepack_size(8960, 1536, 1) == 64 + 8960 * 768 + 8960 * 96 + 8960 * 4
    # tiled: 256-byte header + 576 bytes per (32-row panel, K-group) + zsum + bias per padded row
    assert mb.tiled_size(8960, 1536) == 256 + 280 * 48 * 576 + 2 * 8960 * 4
    assert mb.tiled_size(33, 40) == 256 + 2 * 2 * 576 + 2 * 64 * 4
    assert mb.workspace_size(512, 1536) >= 512 * 1536 + 512 * 8


def test_default_kernel_by_batch_size():
    """Which kernel family the default policy takes (host logic only): the single-launch GEMV up to 4 rows, the
    streaming tensor-core GEMM up to 64 rows where its plan applies (a cluster of at most 8 CTAs must hold the
    activations of a row: K up to 12288 at 64 rows), the tcgen05 tile GEMM above, the dp4a kernel for what is left;
    and the workspace covers the activation blocks of whichever is taken."""
    L = mb.lib()
    for k, n in ((1536, 1536), (1536, 256), (1536, 8960), (8960, 1536), (8192, 28672)):
        for m in (1, 4):
            assert L.mllmb200_w4a32_select_kernel(m, k, n) == mb.KERNEL_GEMV
        for m in (5, 8, 33, 64):
            assert L.mllmb200_w4a32_select_kernel(m, k, n) == mb.KERNEL_STREAM_TC
            assert mb.workspace_size(m, k) >= (k // 32) * ((m + 7) // 8 * 8) * 36 + m * 8
        for m in (65, 512):
            assert L.mllmb200_w4a32_select_kernel(m, k, n) == mb.KERNEL_TC
    assert L.mllmb200_w4a32_select_kernel(64, 32768, 64) in (mb.KERNEL_TC, mb.KERNEL_SIMT)  # a row's activations do not fit 8 CTAs
    assert L.mllmb200_w4a32_select_kernel(8, 32768, 64) == mb.KERNEL_STREAM_TC               # ... but those of 8 rows do


def test_gemv_plan_replay_covers_every_cell_once():
    """The streaming GEMV's work decomposition, replayed on the host with the kernel's own walk: every weight
    cell requested and consumed once, every activation group a CTA reads quantized by it, every panel finished
    once - for the BASELINE shapes (single, grouped, the seven linears of a layer, the 28672 x 8192 matrix and
    its tensor-parallel shards) and for a seeded sweep of odd ones."""
    import random
    layer_k = [1536] * 6 + [8960]
    layer_n = [1536, 256, 256, 1536, 8960, 8960, 1536]
    cases = [(1, [1536], [1536]), (1, [1536] * 3, [1536, 256, 256]), (1, [1536] * 2, [8960, 8960]), (1, [8960], [1536]),
             (1, layer_k, layer_n), (4, layer_k, layer_n), (1, [8192], [28672]), (4, [8192], [28672]),
             (1, [8192], [28672 // 8]), (1, [8192], [28672 // 2]), (2, [1176], [1280]), (1, [33], [40]), (1, [32], [1])]
    for m, ks, ns in cases:
        plan = mb.gemv_plan_check(m, ks, ns)
        assert plan is not None and plan["clusters"] >= 1, (m, ks, ns)
        assert plan["smem"] <= 200 * 1024
    rnd = random.Random(7)
    planned = 0
    for _ in range(300):
        m = rnd.randint(1, 4)
        cnt = rnd.randint(1, 8)
        ks = [rnd.choice([32, 33, 64, 96, 100, 256, 1000, 1536, 4096, 8960, 12000, 20000]) for _ in range(cnt)]
        ns = [rnd.choice([1, 7, 31, 32, 33, 64, 100, 256, 1000, 1536, 5000, 20000]) for _ in range(cnt)]
        planned += mb.gemv_plan_check(m, ks, ns) is not None  # raises when the replay finds a fault
    assert planned > 200
