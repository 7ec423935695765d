"""Tensor-parallel entry points of the C ABI (mllmb200_w4a32_tp_*) on GPUs.

One GPU: a single-rank group goes through the same calls (init, output allocation, forward with every gather mode)
and must reproduce the ordinary forward bit for bit.  Two or more GPUs (skipped when the box has one): two
processes over NCCL, every rank holds half of the rows, and the gathered y - by the fused peer stores and by the
NCCL baseline - must equal the unsharded result computed on the same GPU, for the GEMV (M = 1, 3), the dp4a and int8
tensor-core kernels (pushed to the peers by device copies) and the fp16 tensor-core GEMM (peer stores from its epilogue)."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import mllm_b200 as mb  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def _case(n, k, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32)
    return mb.quant_prepack(w, b)


def test_single_rank_group_equals_ordinary_forward():
    n, k = 512, 1536
    blob = _case(n, k, 1)
    full = mb.W4A32Weights.from_blob(blob)
    h, y = C.c_void_p(), C.c_void_p()
    L = mb.lib()
    assert L.mllmb200_w4a32_tp_init(1, 0, None, C.byref(h)) == 0
    try:
        assert L.mllmb200_w4a32_tp_alloc_output(h, 256 * n * 4, C.byref(y), None) == 0
        from mllm_b200.tp import _DevArray
        ws = torch.empty(mb.workspace_size(256, k), dtype=torch.uint8, device="cuda")
        for m, kern in ((1, 0), (3, 0), (8, 0), (64, 0), (200, 5)):
            x = torch.randn((m, k), device="cuda")
            ref = mb.linear_forward(x, full, kernel=kern)
            for mode in (0, 2):
                out = torch.as_tensor(_DevArray(y.value, (m, n)), device="cuda")
                out.fill_(float("nan"))
                st = L.mllmb200_w4a32_linear_forward_tp(h, x.data_ptr(), full.tiled.data_ptr(), ws.data_ptr(), m, k, n, k, kern,
                                                        mode, None)
                assert st == 0, mb.status_str(st)
                torch.cuda.synchronize()
                mb.check_device_status()
                assert torch.equal(out, ref), (m, kern, mode)
    finally:
        L.mllmb200_w4a32_tp_destroy(h)


def test_tp_argument_checks():
    L = mb.lib()
    h = C.c_void_p()
    assert L.mllmb200_w4a32_tp_init(0, 0, None, C.byref(h)) == 1
    assert L.mllmb200_w4a32_tp_init(9, 0, None, C.byref(h)) == 1
    assert L.mllmb200_w4a32_tp_init(2, 2, None, C.byref(h)) == 1
    assert L.mllmb200_w4a32_tp_init(2, 0, None, C.byref(h)) == 0  # without a communicator: peers by ipc_export / ipc_import
    y = C.c_void_p()
    assert L.mllmb200_w4a32_tp_alloc_output(h, 1024, C.byref(y), None) == 1  # needs the communicator for 2 ranks
    L.mllmb200_w4a32_tp_destroy(h)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, results):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "mllm-advanced_b200"))
    import torch.distributed as dist
    import mllm_b200 as mbw
    from mllm_b200 import tp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = True
    try:
        n, k = 1024, 1536
        blob = _case(n, k, 5)  # the same on every rank
        full = mbw.W4A32Weights.from_blob(blob)
        tpl = tp.TensorParallelLinear(blob, 256)
        g = torch.Generator(device="cuda").manual_seed(11)
        for m, kern in ((1, 0), (3, 0), (8, 0), (64, 0), (200, 5), (256, 4)):
            x = torch.randn((m, k), device="cuda", generator=g)
            ref = mbw.linear_forward(x, full, kernel=kern)
            for mode in (tp.GATHER_PEER_STORES, tp.GATHER_NCCL):
                tpl.output(m).fill_(float("nan"))
                torch.cuda.synchronize()
                dist.barrier()
                y = tpl.forward(x, gather=mode, kernel=kern)
                torch.cuda.synchronize()
                mbw.check_device_status()
                if m <= 4 or kern in (4, 5):
                    # the GEMV shard splits K over its CTAs differently from the full matrix, and the fp16 tile GEMM
                    # splits K in two on launches that fill under half of the GPU and on the tiles left over after
                    # a launch's last full wave - which tiles those are differs between the full matrix and its
                    # shards: other orders of the same fp32 additions
                    rms = float(ref.pow(2).mean().sqrt())
                    good = float((y - ref).abs().max()) <= 1e-5 * rms
                else:
                    good = bool(torch.equal(y, ref))
                if mode == tp.GATHER_PEER_STORES:
                    y_fused = y.clone()
                else:  # both gather modes move the same shard results
                    good = good and bool(torch.equal(y, y_fused))
                ok = ok and good
                dist.barrier()
        tpl.close()
    finally:
        results[rank] = ok
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_fused_gather_and_nccl_match_unsharded():
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), results), nprocs=2, join=True)
    assert all(results.get(r) is True for r in range(2)), dict(results)
