"""World-size-2 test of the column-sharded path on CPU (gloo): shard arithmetic, the all-gather
layout and its un-permutation.  The per-rank GEMM is stood in for by the oracle (test
infrastructure); on GPUs the same code runs the CUDA plan (bench.py --gpus N)."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, M, N, K, ret):
    import torch
    import torch.distributed as dist
    from blaze_b200 import sharded
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng_a, rng_b = np.random.default_rng(42), np.random.default_rng(123)
        ad, asf, ga = O.quantize_nvfp4(rng_a.standard_normal((M, K)).astype(np.float32))       # replicated
        bd, bsf, gb = O.quantize_nvfp4(rng_b.standard_normal((N, K)).astype(np.float32))       # then sharded
        lo, hi = sharded.shard_bounds(N, world, rank)
        bd_r, bsf_r = sharded.shard_weights(bd, bsf, N, world, rank)
        assert bd_r.shape == (N // world, K // 2) and bsf_r.shape == (N // world, K // 16)
        acc, alpha = O.gemm_nvfp4(ad, asf, ga, bd_r, bsf_r, gb, nthreads=2)
        c_local = torch.from_numpy(O.narrow(O.epilogue(acc, alpha), "bf16").astype(np.int16)).view(torch.bfloat16)
        gathered = sharded.all_gather_output(c_local)
        assert tuple(gathered.shape) == (world, M, N // world)
        full = sharded.gathered_to_full(gathered)
        if rank == 0:
            acc_f, alpha_f = O.gemm_nvfp4(ad, asf, ga, bd, bsf, gb, nthreads=2)
            want = O.narrow(O.epilogue(acc_f, alpha_f), "bf16")
            got = full.view(torch.int16).numpy().view(np.uint16)
            ret["equal"] = bool(np.array_equal(got, want))
            ret["block"] = bool(np.array_equal(gathered[1].view(torch.int16).numpy().view(np.uint16), want[:, N // world:]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_column_sharding_two_ranks_gloo():
    import torch.multiprocessing as mp
    from oracle import build_oracle
    build_oracle.build_oracle()
    world, M, N, K = 2, 16, 512, 256
    port = _free_port()
    mgr = mp.Manager(); ret = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, ret)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(120) for p in procs]
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert ret.get("equal") is True and ret.get("block") is True


def test_shard_bounds_errors():
    from blaze_b200 import sharded
    assert sharded.shard_bounds(28672, 8, 3) == (3 * 3584, 4 * 3584)
    assert sharded.shard_bounds(28672, 1, 0) == (0, 28672)
    with pytest.raises(ValueError):
        sharded.shard_bounds(1000, 3, 0)
    with pytest.raises(ValueError):
        sharded.shard_bounds(1024, 2, 2)
    with pytest.raises(ValueError):
        sharded.shard_bounds(384, 2, 0)          # 192 per rank is not a multiple of the tile width
