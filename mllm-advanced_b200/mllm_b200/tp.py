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
