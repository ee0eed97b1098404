"""blz_gemm_nvfp4_decode_static -- the entry point for callers that cannot allocate device memory
(a serving runtime whose arena already owns all of HBM; a loop that cannot take cudaMalloc's
synchronisation).  It must give exactly what the plan-based decode path gives, on two calls in a
row that share the library's fixed workspace (different inputs, so stale partial sums or counters
from the first call would show in the second).  Collected last on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(oracle, device, M, N, K, seed):
    import torch
    from blaze_b200 import GemmPlan, tile_scales
    rng = np.random.default_rng(seed)
    ad, asf, ga = oracle.quantize_nvfp4(rng.standard_normal((M, K)).astype(np.float32))
    bd, bsf, gb = oracle.quantize_nvfp4(rng.standard_normal((N, K)).astype(np.float32))
    u8 = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.uint8)).to(device)
    tA, tB = u8(ad), u8(bd)
    tAs, tBs = tile_scales(u8(asf), M, K), tile_scales(u8(bsf), N, K)
    ref = torch.full((M, N), -3.0, dtype=torch.bfloat16, device=device)
    plan = GemmPlan("nvfp4", M, N, K, tA, tB, A_sf=tAs, B_sf=tBs, a_scale=ga, b_scale=gb, out_dtype="bf16",
                    a_sf_layout="tiled", b_sf_layout="tiled", variant="decode")
    plan.execute(ref); plan.check()
    split = plan.info()["split_k"]
    plan.destroy()
    return (tA, tAs, ga, tB, tBs, gb), ref, split


def test_static_workspace_entry_point_matches_plan_path(oracle, cuda_device):
    import torch
    from blaze_b200 import gemm_nvfp4_decode_static
    from blaze_b200 import _native as nv
    splits = []
    # two calls in a row; both split K, the second with other shapes and data
    for (M, N, K, seed) in [(16, 4096, 4096, 1), (32, 1024, 2048, 2)]:
        (tA, tAs, ga, tB, tBs, gb), ref, split = _case(oracle, cuda_device, M, N, K, seed)
        splits.append(split)
        out = torch.full((M, N), -5.0, dtype=torch.bfloat16, device=cuda_device)
        status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        gemm_nvfp4_decode_static(tA, tAs, ga, tB, tBs, gb, M, N, K, out, out_dtype="bf16", status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(out, ref), "static-workspace result differs from the plan path for %s" % ((M, N, K),)
    assert min(splits) > 1                                     # the shared partial-sum area was really used
    # sizes beyond the fixed workspace are refused before anything is launched
    L = nv.lib()
    big = L.blz_gemm_nvfp4_decode_static(tA.data_ptr(), tAs.data_ptr(), 1.0, tB.data_ptr(), tBs.data_ptr(), 1.0, 65, 1024, 2048,
                                         out.data_ptr(), nv.BF16, 0, None, None)
    assert big == nv.ERR_TOO_LARGE
    wide = L.blz_gemm_nvfp4_decode_static(tA.data_ptr(), tAs.data_ptr(), 1.0, tB.data_ptr(), tBs.data_ptr(), 1.0, 16, 128 * 1025, 2048,
                                          out.data_ptr(), nv.BF16, 0, None, None)
    assert wide == nv.ERR_TOO_LARGE
