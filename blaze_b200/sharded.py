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


class PeerOutput:
    """A full-width [M, N_total] output on every rank, each visible to every other rank of the box
    (CUDA IPC), for the fused GEMM + all-gather (`GemmPlan.execute_gather`).

    `ptrs[i]` is the address of rank i's buffer as seen from this process; `local` is this rank's
    buffer as a torch tensor.  Call `close()` on every rank before the process group goes away."""

    def __init__(self, M: int, n_total: int, dtype, group=None):
        import ctypes
        import torch
        import torch.distributed as dist
        from . import _native as nv
        self._nv, self._torch = nv, torch
        self.M, self.n_total, self.dtype = int(M), int(n_total), dtype
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        esize = torch.empty((), dtype=dtype).element_size()
        self.bytes = self.M * self.n_total * esize
        L = nv.lib()
        own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        nv.check("blz_peer_buffer_create", L.blz_peer_buffer_create(self.bytes, ctypes.byref(own), handle))
        self._own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs, self._opened = [], []
        for r in range(self.world):
            if r == self.rank:
                self.ptrs.append(self._own)
                continue
            p = ctypes.c_void_p()
            nv.check("blz_peer_buffer_open", L.blz_peer_buffer_open(handles[r], ctypes.byref(p)))
            self.ptrs.append(p.value)
            self._opened.append(p.value)
        typestr = {torch.bfloat16: "<u2", torch.float16: "<f2", torch.float32: "<f4"}[dtype]

        class _Cai:
            __cuda_array_interface__ = {"shape": (self.M, self.n_total), "typestr": typestr, "data": (self._own, False), "version": 3}
        t = torch.as_tensor(_Cai(), device=torch.device("cuda", torch.cuda.current_device()))
        self.local = t.view(torch.bfloat16) if dtype == torch.bfloat16 else t
        dist.barrier(group=group)

    def close(self) -> None:
        L = self._nv.lib()
        self._torch.cuda.synchronize()
        self.local = None
        for p in self._opened:
            L.blz_peer_buffer_close(p)
        self._opened = []
        if self._own:
            L.blz_peer_buffer_destroy(self._own)
            self._own = None
