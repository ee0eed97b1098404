"""blz_gemm_nvfp4_decode_static -- the entry point for callers that cannot allocate device memory
(a serving runtime whose arena already owns all of HBM; a loop that cannot take cudaMalloc's
synchronisation).  Checked against the CPU oracle (the parity bar) and against the plan-based
decode path (a different kernel with the same K partition: bit-identical), on calls in a row that
share the library's fixed workspace -- different inputs each time, so stale partial sums or
counters from one call would show in the next.  Collected last on purpose."""
import numpy as np
import pytest

from helpers import assert_close, torch_to_f32

pytestmark = pytest.mark.gpu

# (M, N, K, out_dtype, extra row pitch, seed).  Back to back on one stream, all through the same array.
CASES = [
    (16, 4096, 4096, "bf16", 0, 1),      # K split across CTAs, 16-row instruction
    (32, 1024, 2048, "bf16", 0, 2),      # other shape and data right behind it: the counters must have been cleared
    (5, 1000, 1056, "bf16", 0, 3),       # M below the instruction rows, ragged last weight tile, ragged last K stage
    (48, 384, 512, "f32", 8, 4),         # 64-row instruction, fp32 output, padded rows
    (16, 22016, 256, "f16", 0, 5),       # more tiles than SMs: no K split, nothing goes through the partial sums
    (64, 640, 4096, "bf16", 0, 6),
]


def _case(oracle, device, M, N, K, out_dtype, pad, seed):
    import torch
    from blaze_b200 import GemmPlan, tile_scales
    rng = np.random.default_rng(seed)
    qa = oracle.quantize_nvfp4(rng.standard_normal((M, K)).astype(np.float32))
    qb = oracle.quantize_nvfp4(rng.standard_normal((N, K)).astype(np.float32))
    (ad, asf, ga), (bd, bsf, gb) = qa, qb
    acc, alpha = oracle.gemm_nvfp4(ad, asf, ga, bd, bsf, gb)
    want = oracle.widen(oracle.narrow(oracle.epilogue(acc, alpha), out_dtype), out_dtype)
    u8 = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.uint8)).to(device)
    tA, tB = u8(ad), u8(bd)
    tAs, tBs = tile_scales(u8(asf), M, K), tile_scales(u8(bsf), N, K)
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[out_dtype]
    ldc = N + pad
    ref = torch.full((M, ldc), -3.0, dtype=dt, device=device)
    plan = GemmPlan("nvfp4", M, N, K, tA, tB, A_sf=tAs, B_sf=tBs, a_scale=ga, b_scale=gb, out_dtype=out_dtype,
                    a_sf_layout="tiled", b_sf_layout="tiled", variant="decode", ldc=ldc)
    plan.execute(ref); plan.check()
    split = plan.info()["split_k"]
    plan.destroy()
    return (tA, tAs, ga, tB, tBs, gb), want, ref, split, dt, ldc


def test_static_workspace_entry_point(oracle, cuda_device, monkeypatch):
    import torch
    from blaze_b200 import gemm_nvfp4_decode_static
    from blaze_b200 import _native as nv
    monkeypatch.delenv("BLZ_DECODE_SPLIT", raising=False)        # both paths read it; the test wants the automatic rule
    prepared = [_case(oracle, cuda_device, *c) for c in CASES]
    outs = [torch.full((c[0], ldc), -5.0, dtype=dt, device=cuda_device) for c, (_, _, _, _, dt, ldc) in zip(CASES, prepared)]
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    # the first call on a device loads the module that holds the array; every later call must leave the
    # device's free memory exactly as it found it
    (tA, tAs, ga, tB, tBs, gb) = prepared[0][0]
    gemm_nvfp4_decode_static(tA, tAs, ga, tB, tBs, gb, *CASES[0][:3], outs[0], out_dtype=CASES[0][3], ldc=prepared[0][5], status=status)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for rep in range(2):                                         # the whole sequence twice, no synchronisation in between
        for c, (ops, _, _, _, _, ldc), out in zip(CASES, prepared, outs):
            (tA, tAs, ga, tB, tBs, gb) = ops
            gemm_nvfp4_decode_static(tA, tAs, ga, tB, tBs, gb, c[0], c[1], c[2], out, out_dtype=c[3], ldc=ldc, status=status)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the allocation-free entry point changed the device's free memory: %d -> %d" % (free_before, free_after)
    assert int(status.item()) == 0
    splits = []
    for c, (_, want, ref, split, _, ldc), out in zip(CASES, prepared, outs):
        M, N, K, out_dtype = c[:4]
        splits.append(split)
        got = torch_to_f32(out[:, :N].contiguous(), oracle, out_dtype)
        assert_close(got, want, "static entry point vs oracle %s" % (c,))
        assert torch.equal(out[:, :N], ref[:, :N]), "static-workspace result differs from the plan path for %s" % (c,)
        if ldc > N:
            assert bool((out[:, N:] == -5.0).all()), "wrote past N for %s" % (c,)
    assert max(splits) > 1 and min(splits) == 1                  # the shared partial sums were used, and the unsplit path too
    # sizes beyond the fixed workspace are refused before anything is launched
    L = nv.lib()
    (tA, tAs, ga, tB, tBs, gb) = prepared[1][0]
    out = outs[1]
    big = L.blz_gemm_nvfp4_decode_static(tA.data_ptr(), tAs.data_ptr(), 1.0, tB.data_ptr(), tBs.data_ptr(), 1.0, 65, 1024, 2048,
                                         out.data_ptr(), nv.BF16, 0, None, None)
    assert big == nv.ERR_TOO_LARGE
    wide = L.blz_gemm_nvfp4_decode_static(tA.data_ptr(), tAs.data_ptr(), 1.0, tB.data_ptr(), tBs.data_ptr(), 1.0, 16, 128 * 1025, 2048,
                                          out.data_ptr(), nv.BF16, 0, None, None)
    assert wide == nv.ERR_TOO_LARGE
