"""Two-GPU test of the fused GEMM + all-gather: every rank's epilogue stores its column block into
every rank's full-width output (TMA stores to peer memory); after a barrier each rank must hold
exactly what the local GEMMs plus an NCCL all-gather give.  Skipped with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from blaze_b200 import GemmPlan, quantize_nvfp4, sharded
        M, N, K = 512, 2048, 1024
        n_local = N // world
        ga = torch.Generator(device=dev).manual_seed(42)
        gb = torch.Generator(device=dev).manual_seed(123)
        xa = torch.randn((M, K), generator=ga, device=dev)                       # replicated activations
        xb_full = torch.randn((N, K), generator=gb, device=dev)                  # same weights on every rank, then sharded
        lo, hi = sharded.shard_bounds(N, world, rank)
        ad, asf, gA = quantize_nvfp4(xa, tiled=True)
        # one global scale for the whole weight matrix, so that shards and the full matrix agree
        bd, bsf, gB = quantize_nvfp4(xb_full, tiled=False)
        bd_r, bsf_r = sharded.shard_weights(bd, bsf, N, world, rank)
        plan = GemmPlan("nvfp4", M, n_local, K, ad, bd_r.contiguous(), A_sf=asf, B_sf=bsf_r.contiguous(), a_scale=float(gA.item()),
                        b_scale=float(gB.item()), a_sf_layout="tiled", out_dtype="bf16", variant="256x256")
        # reference: local GEMM, then NCCL all-gather, then un-permute
        c_local = torch.empty((M, n_local), dtype=torch.bfloat16, device=dev)
        plan.execute(c_local); plan.check()
        want = sharded.gathered_to_full(sharded.all_gather_output(c_local))
        # fused: every rank stores into every rank's full-width buffer
        out = sharded.PeerOutput(M, N, torch.bfloat16)
        out.local.fill_(-3.0)
        torch.cuda.synchronize(); dist.barrier()
        plan.execute_gather(out.ptrs, N, lo)
        plan.check()
        torch.cuda.synchronize(); dist.barrier()
        ok = bool(torch.equal(out.local, want))
        out.close()
        plan.destroy()
        dist.barrier()
        # the same three results through the C-level sharded plan (blz_sharded_plan_*): none / NCCL / peer stores
        kw = dict(A_sf=asf, B_sf=bsf_r.contiguous(), a_scale=float(gA.item()), b_scale=float(gB.item()), a_sf_layout="tiled",
                  out_dtype="bf16", variant="256x256")
        sp = sharded.ShardedPlan("nvfp4", M, N, K, ad, bd_r.contiguous(), exchange="none", **kw)
        assert (sp.col_lo, sp.col_hi) == (lo, hi)
        c2 = torch.empty((M, n_local), dtype=torch.bfloat16, device=dev)
        sp.execute(c2); sp.check()
        ok = ok and bool(torch.equal(c2, c_local))
        sp.destroy()
        sp = sharded.ShardedPlan("nvfp4", M, N, K, ad, bd_r.contiguous(), exchange="nccl", **kw)
        g2 = torch.full((world, M, n_local), -3.0, dtype=torch.bfloat16, device=dev)
        sp.execute(g2); sp.check()
        ok = ok and bool(torch.equal(sharded.gathered_to_full(g2), want))
        sp.destroy()
        dist.barrier()
        sp = sharded.ShardedPlan("nvfp4", M, N, K, ad, bd_r.contiguous(), exchange="peer_stores", **kw)
        sp.output.fill_(-3.0)
        torch.cuda.synchronize(); dist.barrier()
        sp.execute(); sp.check()
        torch.cuda.synchronize(); dist.barrier()
        ok = ok and bool(torch.equal(sp.output, want))
        dist.barrier()
        sp.destroy()
        ret[rank] = ok
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_fused_gather_two_gpus(native_lib):
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    port = _free_port()
    mgr = mp.Manager(); ret = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(300) for p in procs]
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert all(ret.get(r) is True for r in range(world)), dict(ret)
