"""The allocation-free forward (mllmb200_w4a32_linear_forward_static) against the ordinary one.

Some callers of this library cannot allocate device memory when they call it: the host framework
owns all of it through its own pool, or the call sits in a loop where cudaMalloc's device-wide
synchronization is not acceptable.  For them the library keeps the activation workspace in a fixed
1 MiB array of its own.  This test drives that entry point through the C ABI, twice in a row (the
array is shared and keeps the previous call's contents, so the second call must not be disturbed by
the first), and requires the same output as mllmb200_w4a32_linear_forward - bit for bit, since both
run the same kernels, and in any case within the 1e-3 * rms bound the other GPU tests use; one case
is also compared with the CPU oracle so that this file stands on its own.  The second call of every
case must leave the device's free memory where it was (nothing allocated, nothing freed).
It also checks that an oversized request is refused instead of overrunning the array.

The file name sorts last so that a run that stops at the first failure has already run every
other test; the test passes on its own in a fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import mllm_b200 as mb  # noqa: E402


def _static_forward(x, wt, y):
    L = mb.lib()
    fn = L.mllmb200_w4a32_linear_forward_static
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 5 + [C.c_void_p]
    fn.restype = C.c_int
    return fn(x.data_ptr(), wt.tiled.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], wt.n, x.stride(0), y.stride(0),
              C.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_forward_matches_ordinary_forward_twice():
    assert torch.cuda.is_available()
    rng = np.random.default_rng(2024)
    from oracle_lib import Oracle
    orc = Oracle()
    # kernels that keep the quantized activations in the scratch array: dp4a GEMM (M = 8), tensor-core GEMM
    # (M = 48, M = 200); and the single-launch GEMV (M = 1, 4), which needs no scratch but shares the entry point
    cases = [(8, 1536, 2048), (48, 1536, 256), (200, 1536, 256), (1, 1536, 2048), (4, 8960, 1536)]
    for m, k, n in cases:
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        b = (rng.standard_normal(n) * 0.1).astype(np.float32)
        blob = mb.quant_prepack(w, b)
        wt = mb.W4A32Weights.from_blob(blob)
        for call in range(2):  # two calls in a row, different activations each time
            x_np = rng.standard_normal((m, k)).astype(np.float32)
            x = torch.from_numpy(x_np).cuda()
            ref = mb.linear_forward(x, wt)
            y = torch.full((m, n), float("nan"), device="cuda")
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            st = _static_forward(x, wt, y)
            assert st == 0, mb.status_str(st)
            torch.cuda.synchronize()
            if call == 1:  # the first call of the process may load the kernels' code
                assert torch.cuda.mem_get_info()[0] == free_before, (m, k, n)
            mb.check_device_status()
            ref_np, y_np = ref.cpu().numpy(), y.cpu().numpy()
            rms = float(np.sqrt(np.mean(ref_np.astype(np.float64) ** 2)))
            assert np.max(np.abs(y_np - ref_np)) <= 1e-3 * rms, (m, k, n, call)
            assert np.array_equal(y_np, ref_np), (m, k, n, call)
            if m == 8:  # and against the CPU oracle
                q, s, _ = mb.blob_sections(blob)
                want = orc.linear(x_np, np.ascontiguousarray(q), np.ascontiguousarray(s), b)
                assert np.max(np.abs(y_np - want)) <= 1e-3 * rms, (m, k, n, call)


def test_static_forward_rejects_requests_beyond_its_capacity():
    L = mb.lib()
    cap = C.c_size_t()
    L.mllmb200_w4a32_static_scratch_bytes.argtypes = [C.POINTER(C.c_size_t)]
    assert L.mllmb200_w4a32_static_scratch_bytes(C.byref(cap)) == 0
    assert cap.value == 1 << 20
    m, k, n = 512, 8960, 64  # prefill-sized: needs far more than 1 MiB of workspace
    assert mb.workspace_size(m, k) > cap.value
    w = np.zeros((n, k), np.float32)
    wt = mb.W4A32Weights.from_blob(mb.quant_prepack(w))
    x = torch.zeros((m, k), device="cuda")
    y = torch.full((m, n), 7.0, device="cuda")
    assert _static_forward(x, wt, y) == 6  # MLLMB200_TOO_LARGE
    torch.cuda.synchronize()
    assert torch.all(y == 7.0)  # nothing ran
