"""World-size-2 (and 3) CPU test of the tensor-parallel host logic over gloo: shard planning, the
all-gather and the column re-assembly.  The per-shard product is computed by the CPU oracle here (no
GPU in this test); on the GPUs the same code path calls the CUDA forward (bench.py `tp`,
tests/test_gpu_parity.py::test_row_shards_concatenate_to_full_result)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, k, m, results):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "mllm-advanced_b200"))
    from mllm_b200 import tp
    from oracle_lib import Oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = Oracle()
        rng = np.random.default_rng(7)  # same data on every rank: x is replicated, W is sharded by rows
        x = rng.standard_normal((m, k)).astype(np.float32)
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        b = rng.standard_normal(n).astype(np.float32)
        q, s = orc.quant_weights(w)
        full = orc.linear(x, q, s, b)
        shard, plan = tp.shard_rows(n, world)
        r0, cnt = plan[rank]
        y_local = torch.zeros((m, shard), dtype=torch.float32)
        if cnt > 0:
            y_local[:, :cnt] = torch.from_numpy(orc.linear(x, np.ascontiguousarray(q[r0:r0 + cnt]),
                                                           np.ascontiguousarray(s[r0:r0 + cnt]), b[r0:r0 + cnt]))
        y = tp.gather_columns(y_local, n, shard)
        results[rank] = bool(np.array_equal(y.numpy(), full))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 256), (2, 100), (3, 200)])
def test_sharded_linear_allgather_matches_unsharded(world, n):
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), n, 96, 3, results), nprocs=world, join=True)
    assert all(results.get(r) is True for r in range(world)), dict(results)


def test_shard_plan():
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "mllm-advanced_b200"))
    from mllm_b200 import tp
    assert tp.shard_rows(8960, 8) == (1120, [(i * 1120, 1120) for i in range(8)])
    assert tp.shard_rows(28672, 8)[0] == 3584
    per, plan = tp.shard_rows(100, 2)
    assert per == 64 and plan == [(0, 64), (64, 36)]
    per, plan = tp.shard_rows(40, 4)
    assert per == 32 and plan == [(0, 32), (32, 8), (40, 0), (40, 0)]
