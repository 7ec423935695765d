"""Tensor parallelism for the W4A32 linear: output channels (rows of W) are sharded over the ranks,
activations are replicated, and the per-rank outputs are all-gathered.

The path shards naturally along N: a row of W, its group scales, its zero-point sum and its bias
entry are independent of every other row, and the activation quantization is per x row, so each
shard's output is bit-identical to that slice of the unsharded output and no reduction is needed -
one all-gather of y per linear (NCCL on the GPUs, gloo in the CPU tests).  The reference project has
no multi-device path at all; this is new functionality."""


def shard_rows(n, world, multiple=32):
    """Rows per rank: equal shards whose size is a multiple of a panel (32 rows), the tail of the last
    ranks possibly empty.  Returns (shard_size, [(row_begin, row_count) per rank])."""
    per = (n + world - 1) // world
    per = (per + multiple - 1) // multiple * multiple
    plan = []
    for r in range(world):
        b = min(n, r * per)
        plan.append((b, max(0, min(n, b + per) - b)))
    return per, plan


def gather_columns(y_local, n, shard_size, group=None):
    """y_local: [M, shard_size] on every rank (columns beyond the rank's real rows are ignored).
    Returns the full [M, n] on every rank."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m = y_local.shape[0]
    assert y_local.shape[1] == shard_size and y_local.is_contiguous()
    gathered = torch.empty((world, m, shard_size), dtype=y_local.dtype, device=y_local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(gathered, y_local, group=group)
    else:  # gloo (CPU tests): list form
        dist.all_gather([gathered[r] for r in range(world)], y_local, group=group)
    # [world, M, shard] -> [M, world*shard] -> first n columns
    return gathered.permute(1, 0, 2).reshape(m, world * shard_size)[:, :n]


class ShardedW4A32Linear:
    """One rank's shard of a linear, built from the full pre-pack blob (every rank reads the same blob
    and repacks only its rows on its own GPU)."""

    def __init__(self, blob, rank, world, device="cuda"):
        from . import binding as mb
        n, k, _, _ = mb.blob_info(blob)
        self.n, self.k, self.rank, self.world = n, k, rank, world
        self.shard_size, plan = shard_rows(n, world)
        self.row_begin, self.row_count = plan[rank]
        self.weights = None
        if self.row_count > 0:
            self.weights = mb.W4A32Weights.from_blob(blob, device=device, row_begin=self.row_begin, row_count=self.row_count)

    def forward_local(self, x, out=None, **kw):
        import torch
        from . import binding as mb
        if out is None:
            out = torch.zeros((x.shape[0], self.shard_size), dtype=torch.float32, device=x.device)
        if self.weights is not None:
            mb.linear_forward(x, self.weights, out=out[:, :self.row_count], **kw)
        return out

    def forward(self, x, group=None, **kw):
        return gather_columns(self.forward_local(x, **kw), self.n, self.shard_size, group)


GATHER_NONE, GATHER_NCCL, GATHER_PEER_STORES = 0, 1, 2


def nccl_comm_ptr(group=None):
    """The ncclComm_t of a torch process group (as an int), once the group has run a collective."""
    import torch
    import torch.distributed as dist
    pg = group if group is not None else dist.distributed_c10d._get_default_group()
    return pg._get_backend(torch.device("cuda"))._comm_ptr()


class _DevArray:
    """Wraps a raw device pointer for torch.as_tensor (the CUDA array interface)."""

    def __init__(self, ptr, shape, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3}


class TensorParallelLinear:
    """One rank of a column-sharded W4A32 linear driven through the C ABI (mllmb200_w4a32_tp_*): the output buffer
    [max_m, n] lives in memory the library maps into every rank's process, and `forward` returns the full y on
    every rank.  blob: the full pre-pack blob (every rank repacks its own rows)."""

    def __init__(self, blob, max_m, group=None, stream=None):
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import binding as mb
        self.mb = mb
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        n, k, _, _ = mb.blob_info(blob)
        assert n % (32 * self.world) == 0, "equal shards of whole 32-row panels"
        self.n, self.k, self.nl, self.max_m = n, k, n // self.world, max_m
        self.weights = mb.W4A32Weights.from_blob(blob, row_begin=self.rank * self.nl, row_count=self.nl)
        # the communicator exists after the first collective of the group
        dist.all_reduce(torch.zeros(1, device="cuda"), group=group)
        torch.cuda.synchronize()
        h = C.c_void_p()
        mb._check(mb.lib().mllmb200_w4a32_tp_init(self.world, self.rank, C.c_void_p(nccl_comm_ptr(group)), C.byref(h)), "tp_init")
        self.handle = h
        y = C.c_void_p()
        mb._check(mb.lib().mllmb200_w4a32_tp_alloc_output(h, max_m * n * 4, C.byref(y), mb._stream_ptr(stream)), "tp_alloc_output")
        self._y_ptr = y.value
        self.ws = torch.empty(mb.workspace_size(max_m, k), dtype=torch.uint8, device="cuda")

    def output(self, m):
        """The library's output buffer viewed as a [m, n] tensor (no copy)."""
        import torch
        return torch.as_tensor(_DevArray(self._y_ptr, (m, self.n)), device="cuda")

    def forward(self, x, gather=GATHER_PEER_STORES, kernel=0, stream=None, pdl=False):
        import ctypes as C
        m = x.shape[0]
        assert m <= self.max_m and x.shape[1] == self.k and x.stride(1) == 1
        self.mb._check(self.mb.lib().mllmb200_w4a32_linear_forward_tp(
            self.handle, x.data_ptr(), self.weights.tiled.data_ptr(), self.ws.data_ptr(), m, self.k, self.n, x.stride(0),
            kernel | (0x100 if pdl else 0), gather, self.mb._stream_ptr(stream)), "linear_forward_tp")
        return self.output(m)

    def close(self):
        if self.handle:
            self.mb.lib().mllmb200_w4a32_tp_destroy(self.handle)
            self.handle = None
