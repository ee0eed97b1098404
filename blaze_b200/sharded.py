"""Column-sharded GEMM across the GPUs of one box: the only multi-GPU element of the path.

Output columns are independent, so the weight matrix (K-major, [N, K]) and its scale rows are
split by rows across ranks; activations are replicated; every rank runs the ordinary single-GPU
plan on (M, N/world, K).  No collective is part of the GEMM; gathering the bf16 output over NCCL
is an optional step after it.  Blaze itself has no multi-GPU code (no NCCL, cudaSetDevice or peer
copy anywhere in its tree); this file has no counterpart there.
"""
from __future__ import annotations


def shard_bounds(n_total: int, world: int, rank: int, multiple: int = 128) -> tuple[int, int]:
    """Rows [lo, hi) of the [N, K] weight matrix owned by `rank`.  Shards are equal and a multiple
    of `multiple` columns (the tile width) so every rank runs full tiles."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank %d of %d" % (rank, world))
    if n_total % world != 0 or (n_total // world) % multiple != 0:
        raise ValueError("N=%d does not split into %d shards that are multiples of %d" % (n_total, world, multiple))
    per = n_total // world
    return rank * per, (rank + 1) * per


def shard_weights(w_data, w_sf_rowmajor, n_total: int, world: int, rank: int):
    """Slices packed weights [N, K/2] (or [N, K]) and row-major scales [N, K/16] for one rank."""
    lo, hi = shard_bounds(n_total, world, rank)
    return w_data[lo:hi], (w_sf_rowmajor[lo:hi] if w_sf_rowmajor is not None else None)


def all_gather_output(c_local, group=None):
    """NCCL (or gloo) all-gather of the local [M, N/world] output: returns [world, M, N/world]."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m, n_local = c_local.shape
    out = torch.empty((world * m, n_local), dtype=c_local.dtype, device=c_local.device)   # rank blocks stacked along dim 0
    dist.all_gather_into_tensor(out, c_local.contiguous(), group=group)
    return out.view(world, m, n_local)


def gathered_to_full(gathered):
    """[world, M, N/world] -> [M, N] (column blocks in rank order)."""
    world, m, n_local = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, world * n_local)
