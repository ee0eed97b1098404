"""Column-sharded GEMM across the GPUs of one box: the only multi-GPU element of the path.

Output columns are independent, so the weight matrix (K-major, [N, K]) and its scale rows are
split by rows across ranks; activations are replicated; every rank runs the ordinary single-GPU
plan on (M, N/world, K).  No collective is part of the GEMM; assembling the full output on every
GPU is an optional step after it (NCCL all-gather) or inside it (peer stores from the epilogue).
Blaze itself has no multi-GPU code (no NCCL, cudaSetDevice or peer copy anywhere in its tree).

The shard arithmetic, the per-rank plan and both exchanges live in the C library
(blz_shard_bounds, blz_sharded_plan_*); ``ShardedPlan`` mirrors them and uses torch.distributed
only as the channel that carries the NCCL id and the buffer handles between the processes.
"""
from __future__ import annotations

import ctypes


def shard_bounds(n_total: int, world: int, rank: int, multiple: int = 128) -> tuple[int, int]:
    """Rows [lo, hi) of the [N, K] weight matrix owned by `rank`.  Shards are equal and a multiple
    of `multiple` columns (the tile width) so every rank runs full tiles."""
    from . import _native as nv
    lo, hi = ctypes.c_int64(), ctypes.c_int64()
    st = nv.lib().blz_shard_bounds(int(n_total), int(world), int(rank), int(multiple), ctypes.byref(lo), ctypes.byref(hi))
    if st != nv.OK:
        raise ValueError("N=%d does not split into %d shards that are multiples of %d (rank %d)" % (n_total, world, multiple, rank))
    return lo.value, hi.value


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


class ShardedPlan:
    """blz_sharded_plan: this rank's share of C = A x W^T with the output exchange chosen at creation.

    ``exchange``: "none" -> execute(C) fills this rank's [M, N/world] block; "nccl" -> execute(C) fills
    [world, M, N/world] (the library's own NCCL communicator, created here collectively); "peer_stores" ->
    execute() stores into every rank's plan-owned row-major [M, N] output, available as ``output`` after the
    caller's barrier.  `B` / `B_sf` are this rank's rows of the K-major weights; N is the full width."""

    def __init__(self, kind: str, M: int, N: int, K: int, A, B, *, exchange: str = "none", group=None, **desc_kw):
        import torch
        import torch.distributed as dist
        from . import _native as nv
        from .gemm import make_desc
        self._nv, self._torch = nv, torch
        L = nv.lib()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.exchange = exchange
        sd = nv.ShardedDesc()
        sd.gemm = make_desc(kind, M, N, K, A, B, **desc_kw)
        sd.world, sd.rank, sd.exchange, sd.reserved = self.world, self.rank, nv.EXCHANGES[exchange], 0
        self._id = None
        if exchange == "nccl" and self.world > 1:
            ids = [None]
            if self.rank == 0:
                buf = ctypes.create_string_buffer(128)
                nv.check("blz_nccl_unique_id", L.blz_nccl_unique_id(buf))
                ids = [buf.raw]
            dist.broadcast_object_list(ids, src=0, group=group)
            self._id = ctypes.create_string_buffer(ids[0], 128)
            sd.nccl_id = ctypes.cast(self._id, ctypes.c_char_p)
        self._keep = (A, B, desc_kw)
        self._handle = ctypes.c_void_p()
        st = L.blz_sharded_plan_create(ctypes.byref(sd), ctypes.byref(self._handle))
        if st != nv.OK:
            raise nv.BlazeError("blz_sharded_plan_create", st, (L.blz_sharded_last_error() or b"").decode() or L.blz_last_cuda_error_string().decode())
        info = self.info()
        self.col_lo, self.col_hi = info["col_lo"], info["col_hi"]
        self.M, self.N = int(M), int(N)
        self.output = None
        if exchange == "peer_stores":
            h = ctypes.create_string_buffer(64)
            nv.check("blz_sharded_plan_output_handle", L.blz_sharded_plan_output_handle(self._handle, h))
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, h.raw, group=group)
            else:
                handles = [h.raw]
            nv.check("blz_sharded_plan_connect", L.blz_sharded_plan_connect(self._handle, b"".join(handles)))
            out_dtype = desc_kw.get("out_dtype", "bf16")
            dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[out_dtype]
            typestr = {"bf16": "<u2", "f16": "<f2", "f32": "<f4"}[out_dtype]
            own = info["own_output"]

            class _Cai:
                __cuda_array_interface__ = {"shape": (self.M, self.N), "typestr": typestr, "data": (own, False), "version": 3}
            t = torch.as_tensor(_Cai(), device=torch.device("cuda", torch.cuda.current_device()))
            self.output = t.view(dt) if dt == torch.bfloat16 else t
            if self.world > 1:
                dist.barrier(group=group)

    def info(self) -> dict:
        i = self._nv.ShardedInfo()
        self._nv.check("blz_sharded_plan_info", self._nv.lib().blz_sharded_plan_info(self._handle, ctypes.byref(i)))
        d = {k: getattr(i, k) for k in ("col_lo", "col_hi", "exchange", "world", "rank", "own_output")}
        d["gemm"] = {name: getattr(i.gemm, name) for name, _ in self._nv.PlanInfo._fields_}
        return d

    def execute(self, C=None, stream=None) -> None:
        from .gemm import _ptr, _stream
        self._nv.check("blz_sharded_plan_execute", self._nv.lib().blz_sharded_plan_execute(self._handle, _ptr(C), _stream(stream)))

    def check(self, stream=None) -> None:
        from .gemm import _stream
        self._nv.check("blz_sharded_plan_check", self._nv.lib().blz_sharded_plan_check(self._handle, _stream(stream)))

    def destroy(self) -> None:
        if self._handle:
            self._torch.cuda.synchronize()
            self.output = None
            self._nv.lib().blz_sharded_plan_destroy(self._handle)
            self._handle = ctypes.c_void_p()
