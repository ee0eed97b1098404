"""GPU parity tests: the CUDA path through the C ABI against the CPU oracle on the same seeded
inputs.  Tolerance: |c - ref| / max(|ref|, 1) <= 1e-2 per element (fp32 accumulation, 16-bit or
fp32 output); byte-level work (quantisers, scale tiling, repacking) must be bit-exact.
Seeds follow Blaze's tests: 42 for A / activations, 123 for B / weights (tests/test_gemm.cu:130-131).
"""
import os
import subprocess

import numpy as np
import pytest

from helpers import assert_close, bits16_to_torch, torch_to_f32

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def _torch():
    import torch
    return torch


def _out_tensor(M, N, out_dtype, device, ldc=0):
    torch = _torch()
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[out_dtype]
    return torch.full((M, ldc or N), -7.0, dtype=dt, device=device)


def _u8(a, device):
    return _torch().from_numpy(np.ascontiguousarray(a, np.uint8)).to(device)


def _run(plan, C):
    plan.execute(C)
    plan.check()
    return C


# --------------------------------------------------------------------------- dense fp16 / bf16

def _dense_inputs(oracle, kind, M, N, K, scale=1.0):
    rng_a, rng_b = np.random.default_rng(42), np.random.default_rng(123)
    enc = oracle.f32_to_f16 if kind == "f16" else oracle.f32_to_bf16
    A = enc((rng_a.standard_normal((M, K)) * scale).astype(np.float32))
    Bt = enc((rng_b.standard_normal((N, K)) * scale).astype(np.float32))
    return A, Bt


@pytest.mark.parametrize("kind,out_dtype,variant,shape", [
    ("f16", "f32", "128x128", (128, 128, 64)),       # one tile, one K stage
    ("f16", "f32", "128x128", (128, 128, 256)),      # one tile, four K stages
    ("f16", "f32", "128x128", (256, 256, 256)),      # the 256^3 fp16 configuration
    ("bf16", "bf16", "128x128", (256, 384, 512)),
    ("bf16", "bf16", "256x256", (256, 512, 192)),
    ("f16", "f16", "256x256", (384, 768, 1024)),
    ("bf16", "f32", "auto", (300, 200, 136)),        # ragged in M, N and K
    ("f16", "bf16", "auto", (1, 128, 64)),           # single row
    ("bf16", "bf16", "256x256", (129, 520, 72)),     # ragged tiles, 256-wide variant
    ("bf16", "bf16", "auto", (2048, 2304, 1024)),    # several tiles per CTA: ring wrap, both accumulators
    ("bf16", "bf16", "256x256", (256, 256, 64)),     # CTA pair, one tile, one K stage
    ("bf16", "bf16", "256x256", (512, 512, 256)),
    ("f16", "f32", "256x256", (300, 520, 136)),      # CTA pair, ragged in M, N and K
    ("f16", "f16", "256x256", (2048, 2304, 1024)),   # CTA pair, several tiles per pair
    ("bf16", "bf16", "128x128", (2048, 1152, 512)),
    ("bf16", "bf16", "512x256", (512, 256, 64)),     # two pairs sharing B, one tile, one K stage
    ("bf16", "f32", "512x256", (700, 520, 392)),     # ragged; the second pair partly outside M
    ("f16", "f16", "512x256", (2048, 2304, 1024)),
    ("bf16", "bf16", "256x128", (256, 128, 64)),     # CTA pair on a 256x128 tile: one tile, one K stage
    ("f16", "f32", "256x128", (300, 200, 136)),      # ... ragged in M, N and K
    ("f16", "f16", "256x128", (2048, 2304, 1024)),   # ... several tiles per pair, the eight-stage ring wraps
    ("f16", "f32", "decode", (1, 128, 64)),          # skinny-M weight stream: one tile, one K stage
    ("bf16", "bf16", "decode", (16, 384, 520)),      # ragged K stage
    ("f16", "f16", "decode", (33, 1000, 1032)),      # 64-row instruction, ragged N
    ("bf16", "f32", "decode", (64, 4096, 4096)),     # K split across a cluster
    ("bf16", "bf16", "decode", (5, 512, 8192)),      # deep K split, ring wraps
    ("bf16", "bf16", "decode", (128, 512, 520)),     # 128-row activation tile, chunked epilogue
    ("f16", "f32", "decode", (65, 384, 4096)),       # the same with a K split
    ("f16", "f16", "decode", (100, 4096, 1024)),
])
def test_dense16(oracle, cuda_device, kind, out_dtype, variant, shape):
    from blaze_b200 import GemmPlan
    M, N, K = shape
    A, Bt = _dense_inputs(oracle, kind, M, N, K)
    ref = oracle.gemm_dense16(A, Bt, kind)
    tA, tB = bits16_to_torch(A, kind, cuda_device), bits16_to_torch(Bt, kind, cuda_device)
    C = _out_tensor(M, N, out_dtype, cuda_device)
    plan = GemmPlan(kind, M, N, K, tA, tB, out_dtype=out_dtype, variant=variant)
    _run(plan, C)
    got = torch_to_f32(C, oracle, out_dtype)
    want = oracle.widen(oracle.narrow(ref, out_dtype), out_dtype)
    assert_close(got, want, "dense %s %s %s %s" % (kind, out_dtype, variant, shape))
    plan.destroy()


def test_fp16_config1_golden(oracle, cuda_device):
    """The 256^3 fp16 configuration: fp16 256^3, A row-major, B column-major, seeded fill 42 / 123, fp32 out,
    checked against the rows Blaze's own gemm_cpu_fp16 produced (tests/golden)."""
    from blaze_b200 import create_fp16_gemm_plan, destroy_fp16_gemm_plan, execute_fp16_gemm
    g = np.load(os.path.join(GOLDEN, "ref_gemm_cpu_fp16_256.npz"))
    M = N = K = 256
    A = oracle.f32_to_f16(oracle.fill_uniform_rand(M * K, 42)).reshape(M, K)
    B = oracle.f32_to_f16(oracle.fill_uniform_rand(K * N, 123)).reshape(K, N)
    tA = bits16_to_torch(A, "f16", cuda_device)
    tB = bits16_to_torch(np.ascontiguousarray(B.T), "f16", cuda_device)      # column-major B = [N, K] rows
    C = _out_tensor(M, N, "f32", cuda_device)
    plan = create_fp16_gemm_plan(tA, tB, M, N, K)
    execute_fp16_gemm(plan, C)
    plan.check()
    got = C.cpu().numpy()
    assert_close(got[g["rows"]], g["C_rows"], "config 1 vs golden rows")
    ref = oracle.gemm_f32(oracle.f16_to_f32(A), np.ascontiguousarray(oracle.f16_to_f32(B).T))
    assert_close(got, ref, "config 1 vs oracle")
    destroy_fp16_gemm_plan(plan)


def test_golden_small_through_cuda(oracle, cuda_device):
    from blaze_b200 import GemmPlan
    g = np.load(os.path.join(GOLDEN, "ref_gemm_cpu_fp16_48x80x96.npz"))
    A, B, Cref = g["A"], g["B"], g["C"]
    M, K = A.shape; N = B.shape[1]
    tA = bits16_to_torch(A, "f16", cuda_device)
    tB = bits16_to_torch(B, "f16", cuda_device)                                # Blaze's [K, N] layout
    C = _out_tensor(M, N, "f32", cuda_device)
    plan = GemmPlan("f16", M, N, K, tA, tB, out_dtype="f32", b_layout="nmajor")
    _run(plan, C)
    assert_close(C.cpu().numpy(), Cref, "golden 48x80x96, B given [K,N]")
    plan.destroy()


# --------------------------------------------------------------------------------------- FP8

def _fp8_inputs(oracle, M, N, K):
    rng_a, rng_b = np.random.default_rng(42), np.random.default_rng(123)
    xa = rng_a.uniform(-1, 1, (M, K)).astype(np.float32)
    xb = rng_b.uniform(-1, 1, (N, K)).astype(np.float32)
    qa, sa = oracle.quantize_fp8(xa)
    qb, sb = oracle.quantize_fp8(xb)
    return qa, float(np.float32(1.0) / np.float32(sa)), qb, float(np.float32(1.0) / np.float32(sb))


@pytest.mark.parametrize("variant,shape", [
    ("128x128", (128, 128, 128)),
    ("128x128", (256, 256, 512)),
    ("256x256", (256, 512, 384)),
    ("auto", (200, 328, 144)),
    ("auto", (32, 4096, 1024)),
    ("256x256", (1024, 2048, 2048)),
    ("256x256", (256, 256, 128)),
    ("256x256", (512, 768, 512)),
    ("256x256", (200, 328, 144)),
    ("256x256", (1024, 2048, 2048)),
    ("512x256", (512, 256, 128)),
    ("512x256", (1024, 2048, 2048)),
    ("512x256", (300, 328, 144)),
    ("256x128", (256, 128, 128)),
    ("256x128", (300, 328, 144)),
    ("256x128", (1024, 2048, 2048)),
    ("decode", (1, 256, 128)),
    ("decode", (32, 4096, 1024)),
    ("decode", (48, 1000, 1136)),
    ("decode", (7, 4096, 11008)),
    ("decode", (64, 12288, 4096)),
    ("decode", (128, 4096, 4096)),                   # 128-row activation tile, K split
    ("decode", (100, 1000, 1136)),
    ("decode", (128, 4096, 11008)),
])
def test_fp8(oracle, cuda_device, variant, shape):
    from blaze_b200 import GemmPlan
    M, N, K = shape
    qa, da, qb, db = _fp8_inputs(oracle, M, N, K)
    acc = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qb))
    alpha = float(np.float32(da) * np.float32(db))
    want = oracle.widen(oracle.narrow(oracle.epilogue(acc, alpha), "bf16"), "bf16")
    C = _out_tensor(M, N, "bf16", cuda_device)
    plan = GemmPlan("fp8", M, N, K, _u8(qa, cuda_device), _u8(qb, cuda_device), a_scale=da, b_scale=db, out_dtype="bf16", variant=variant)
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, "bf16"), want, "fp8 %s %s" % (variant, shape))
    plan.destroy()


def test_fp8_config2_sampled(oracle, cuda_device):
    """The FP8 configuration (4096^3, uniform[-1,1], per-tensor scales to 448, bf16 out): inputs are
    quantised on the GPU (bit-checked against the oracle on a slice), 48 output rows are checked."""
    torch = _torch()
    from blaze_b200 import GemmPlan, quantize_fp8
    M = N = K = 4096
    ga = torch.Generator(device=cuda_device).manual_seed(42)
    gb = torch.Generator(device=cuda_device).manual_seed(123)
    xa = torch.rand((M, K), generator=ga, device=cuda_device) * 2 - 1
    xb = torch.rand((N, K), generator=gb, device=cuda_device) * 2 - 1
    qa, sca = quantize_fp8(xa)
    qb, scb = quantize_fp8(xb)
    sca, scb = sca.cpu().numpy(), scb.cpu().numpy()
    # quantiser parity on the first rows
    s_ref = np.float32(448.0) / np.float32(xa.abs().max().item())
    assert np.float32(sca[0]) == s_ref
    assert np.array_equal(qa[:8].cpu().numpy(), oracle.f32_to_e4m3(xa[:8].cpu().numpy() * s_ref))
    C = _out_tensor(M, N, "bf16", cuda_device)
    plan = GemmPlan("fp8", M, N, K, qa, qb, a_scale=float(sca[1]), b_scale=float(scb[1]), out_dtype="bf16")
    _run(plan, C)
    rows = np.array(sorted(set(np.random.default_rng(5).integers(0, M, 46).tolist() + [0, M - 1])))
    acc = oracle.gemm_f32(oracle.e4m3_to_f32(qa[rows].cpu().numpy()), oracle.e4m3_to_f32(qb.cpu().numpy()))
    alpha = float(np.float32(sca[1]) * np.float32(scb[1]))
    want = oracle.widen(oracle.narrow(oracle.epilogue(acc, alpha), "bf16"), "bf16")
    got = torch_to_f32(C[torch.from_numpy(rows).to(cuda_device)], oracle, "bf16")
    assert_close(got, want, "fp8 config 2 sampled rows")
    plan.destroy()


# ------------------------------------------------------------------------------------- NVFP4

def _nvfp4_inputs(oracle, M, N, K, w_std=1.0):
    rng_a, rng_b = np.random.default_rng(42), np.random.default_rng(123)
    xa = rng_a.standard_normal((M, K)).astype(np.float32)
    xb = (rng_b.standard_normal((N, K)) * w_std).astype(np.float32)
    return oracle.quantize_nvfp4(xa), oracle.quantize_nvfp4(xb)


def _nvfp4_ref(oracle, qa, qb, out_dtype="bf16", **epi):
    (ad, asf, ga), (bd, bsf, gb) = qa, qb
    acc, alpha = oracle.gemm_nvfp4(ad, asf, ga, bd, bsf, gb)
    return oracle.widen(oracle.narrow(oracle.epilogue(acc, alpha, **epi), out_dtype), out_dtype)


@pytest.mark.parametrize("variant,shape", [
    ("128x128", (128, 128, 256)),      # one tile, one K stage
    ("128x128", (128, 128, 1024)),     # one tile, four K stages
    ("128x128", (256, 384, 512)),
    ("256x256", (128, 256, 256)),
    ("256x256", (384, 768, 1536)),
    ("auto", (200, 328, 160)),         # ragged M, N; K not a multiple of the 256-value stage
    ("256x256", (129, 520, 96)),
    ("128x128", (100, 72, 64)),
    ("auto", (1024, 4096, 2048)),
    ("256x256", (2048, 2304, 1024)),   # several tiles per CTA
    ("256x256", (256, 256, 256)),      # CTA pair: one tile, one K stage
    ("256x256", (256, 256, 2048)),     # CTA pair: the stage ring wraps
    ("256x256", (512, 768, 1536)),
    ("256x256", (200, 328, 160)),      # CTA pair, ragged
    ("256x256", (129, 520, 96)),
    ("256x256", (2048, 2304, 1024)),   # several tiles per pair
    ("128x128", (2048, 1152, 1024)),
    ("512x256", (512, 256, 256)),      # two pairs sharing B: one tile, one K stage
    ("512x256", (512, 256, 2048)),     # ... the stage ring wraps
    ("512x256", (1024, 768, 1536)),
    ("512x256", (700, 328, 160)),      # ragged
    ("512x256", (2048, 2304, 1024)),
    ("256x128", (256, 128, 256)),      # CTA pair on a 256x128 tile: one tile, one K stage
    ("256x128", (200, 328, 160)),      # ... ragged
    ("256x128", (2048, 2304, 2048)),   # ... several tiles per pair
    ("decode", (16, 512, 1024)),
    ("decode", (1, 128, 256)),
    ("decode", (7, 200, 160)),
    ("decode", (32, 1024, 2048)),
    ("decode", (64, 640, 4096)),
    ("decode", (16, 4096, 4096)),      # split-K across CTAs
])
def test_nvfp4(oracle, cuda_device, variant, shape):
    from blaze_b200 import GemmPlan
    M, N, K = shape
    qa, qb = _nvfp4_inputs(oracle, M, N, K)
    want = _nvfp4_ref(oracle, qa, qb)
    (ad, asf, ga), (bd, bsf, gb) = qa, qb
    C = _out_tensor(M, N, "bf16", cuda_device)
    plan = GemmPlan("nvfp4", M, N, K, _u8(ad, cuda_device), _u8(bd, cuda_device), A_sf=_u8(asf, cuda_device), B_sf=_u8(bsf, cuda_device),
                    a_scale=ga, b_scale=gb, out_dtype="bf16", variant=variant)
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, "bf16"), want, "nvfp4 %s %s %s" % (variant, shape, plan.info()))
    plan.destroy()


@pytest.mark.parametrize("variant,M", [("128x128", 128), ("256x256", 256), ("256x256", 128), ("256x384", 256), ("256x128", 256), ("decode", 16)])
def test_nvfp4_position_coded(oracle, cuda_device, variant, M):
    """Catches transposition, nibble order and scale-layout errors that constant fills hide:
    row m of A is one-hot at k = (37*m + 5) % K with its own block scale, every weight and every
    weight scale differs, so C[m, n] singles out one element and one scale of B."""
    from blaze_b200 import GemmPlan
    N, K = 256, 512
    codes = np.array([1, 2, 3, 4, 5, 6, 7, 9, 10, 11, 12, 13, 14, 15], np.uint8)
    a_nib = np.zeros((M, K), np.uint8)
    a_sf = np.full((M, K // 16), 0x38, np.uint8)
    for m in range(M):
        k = (37 * m + 5) % K
        a_nib[m, k] = codes[m % len(codes)]
        a_sf[m, k // 16] = 0x30 + (m % 24)
    rng = np.random.default_rng(3)
    b_nib = rng.integers(0, 16, (N, K)).astype(np.uint8)
    b_sf = (0x28 + rng.integers(0, 32, (N, K // 16))).astype(np.uint8)
    pack = lambda nib: (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    ad, bd = pack(a_nib), pack(b_nib)
    want = _nvfp4_ref(oracle, (ad, a_sf, 1.0), (bd, b_sf, 0.5), out_dtype="f32")
    C = _out_tensor(M, N, "f32", cuda_device)
    plan = GemmPlan("nvfp4", M, N, K, _u8(ad, cuda_device), _u8(bd, cuda_device), A_sf=_u8(a_sf, cuda_device), B_sf=_u8(b_sf, cuda_device),
                    a_scale=1.0, b_scale=0.5, out_dtype="f32", variant=variant)
    _run(plan, C)
    got = C.cpu().numpy()
    assert np.array_equal(got, want), "position-coded NVFP4 (%s): %d of %d elements differ" % (variant, int((got != want).sum()), got.size)
    plan.destroy()


@pytest.mark.parametrize("N,K", [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)])
def test_nvfp4_config3_decode(oracle, cuda_device, N, K):
    """The NVFP4 decode configuration: Llama-7B decode projections at M = 16, N(0,1) both sides, bf16 out."""
    from blaze_b200 import GemmPlan
    M = 16
    qa, qb = _nvfp4_inputs(oracle, M, N, K)
    want = _nvfp4_ref(oracle, qa, qb)
    (ad, asf, ga), (bd, bsf, gb) = qa, qb
    C = _out_tensor(M, N, "bf16", cuda_device)
    plan = GemmPlan("nvfp4", M, N, K, _u8(ad, cuda_device), _u8(bd, cuda_device), A_sf=_u8(asf, cuda_device), B_sf=_u8(bsf, cuda_device),
                    a_scale=ga, b_scale=gb, out_dtype="bf16")
    assert plan.info()["variant"] == 3
    _run(plan, C)
    first = C.clone()
    assert_close(torch_to_f32(C, oracle, "bf16"), want, "config 3 decode N=%d K=%d %s" % (N, K, plan.info()))
    for _ in range(3):                                   # run-to-run bit-identical (ordered split-K sum)
        C.fill_(0)
        _run(plan, C)
        assert _torch().equal(C, first)
    plan.destroy()


def test_nvfp4_blaze_layout_and_known_answer(oracle, cuda_device):
    """Blaze's own block-scaled test (tests/test_gemm.cu:338-389): data 0x22, scales 0x38, tensor
    scale 1 => every output equals K, through the Blaze-named API with B given as [K, N/2]."""
    torch = _torch()
    import blaze_b200 as bz
    for (M, N, K) in [(1, 4096, 4096), (32, 512, 1024), (128, 256, 11008), (512, 768, 512)]:
        A = {"data": torch.full((M, K // 2), 0x22, dtype=torch.uint8, device=cuda_device),
             "block_scales": torch.full((M, K // 16), 0x38, dtype=torch.uint8, device=cuda_device), "tensor_scale": 1.0}
        B = {"data": torch.full((K, N // 2), 0x22, dtype=torch.uint8, device=cuda_device),
             "block_scales": torch.full((K // 16, N), 0x38, dtype=torch.uint8, device=cuda_device), "tensor_scale": 1.0}
        C = _out_tensor(M, N, "f16", cuda_device)
        for create, execute, destroy in [
                (bz.create_fp4_blkscaled_gemm_plan, bz.execute_fp4_blkscaled_gemm, bz.destroy_fp4_blkscaled_gemm_plan),
                (bz.create_fp4_blkscaled_persistent_gemm_plan, bz.execute_fp4_blkscaled_persistent_gemm, bz.destroy_fp4_blkscaled_persistent_gemm_plan)]:
            plan = create(A, B, M, N, K)
            execute(plan, C)
            plan.check()
            got = C.float().cpu().numpy()
            assert np.abs(got - K).max() / max(K, 1) < 0.01, (M, N, K, got[0, :4])
            destroy(plan)


def test_nvfp4_nmajor_weights(oracle, cuda_device):
    """B in Blaze's convention: data [K, N/2] (two N-neighbours per byte), scales [K/16, N]."""
    from blaze_b200 import GemmPlan
    M, N, K = 96, 384, 512
    qa, qb = _nvfp4_inputs(oracle, M, N, K)
    want = _nvfp4_ref(oracle, qa, qb)
    (ad, asf, ga), (bd, bsf, gb) = qa, qb
    nib = np.empty((N, K), np.uint8); nib[:, 0::2] = bd & 15; nib[:, 1::2] = bd >> 4
    nib_kn = np.ascontiguousarray(nib.T)                                      # [K, N]
    b_kn = (nib_kn[:, 0::2] | (nib_kn[:, 1::2] << 4)).astype(np.uint8)        # [K, N/2]
    sf_kn = np.ascontiguousarray(bsf.T)                                       # [K/16, N]
    C = _out_tensor(M, N, "bf16", cuda_device)
    plan = GemmPlan("nvfp4", M, N, K, _u8(ad, cuda_device), _u8(b_kn, cuda_device), A_sf=_u8(asf, cuda_device), B_sf=_u8(sf_kn, cuda_device),
                    a_scale=ga, b_scale=gb, out_dtype="bf16", b_layout="nmajor")
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, "bf16"), want, "nvfp4 with [K,N] weights")
    plan.destroy()


def test_nvfp4_config5_sampled(oracle, cuda_device):
    """The sharded NVFP4 configuration on one GPU (M=8192, N=28672, K=8192): operands quantised on the GPU,
    24 rows of the output checked against the oracle, plus a linearity property at full size:
    doubling the activations' tensor scale doubles every output bit-exactly (bf16 keeps exponent)."""
    torch = _torch()
    from blaze_b200 import GemmPlan, quantize_nvfp4
    M, N, K = 8192, 28672, 8192
    ga = torch.Generator(device=cuda_device).manual_seed(42)
    gb = torch.Generator(device=cuda_device).manual_seed(123)
    xa = torch.randn((M, K), generator=ga, device=cuda_device)
    ad, asf, gA = quantize_nvfp4(xa, tiled=False); del xa
    xb = torch.randn((N, K), generator=gb, device=cuda_device)
    bd, bsf, gB = quantize_nvfp4(xb, tiled=False); del xb
    gA, gB = float(gA.item()), float(gB.item())
    C = _out_tensor(M, N, "bf16", cuda_device)
    plan = GemmPlan("nvfp4", M, N, K, ad, bd, A_sf=asf, B_sf=bsf, a_scale=gA, b_scale=gB, out_dtype="bf16")
    _run(plan, C)
    rows = np.array(sorted(set(np.random.default_rng(9).integers(0, M, 22).tolist() + [0, M - 1])))
    ridx = torch.from_numpy(rows).to(cuda_device)
    acc, alpha = oracle.gemm_nvfp4(ad[ridx].cpu().numpy(), asf[ridx].cpu().numpy(), gA, bd.cpu().numpy(), bsf.cpu().numpy(), gB)
    want = oracle.widen(oracle.narrow(oracle.epilogue(acc, alpha), "bf16"), "bf16")
    assert_close(torch_to_f32(C[ridx], oracle, "bf16"), want, "config 5 sampled rows")
    C2 = _out_tensor(M, N, "bf16", cuda_device)
    plan2 = GemmPlan("nvfp4", M, N, K, ad, bd, A_sf=asf, B_sf=bsf, a_scale=2 * gA, b_scale=gB, out_dtype="bf16")
    _run(plan2, C2)
    assert torch.equal(C2, C * 2)
    plan.destroy(); plan2.destroy()


# ------------------------------------------------------------------------------------- W4A16

@pytest.mark.parametrize("kind,shape", [
    ("w4a16_bf16", (129, 256, 512)), ("w4a16_f16", (200, 328, 160)), ("w4a16_bf16", (512, 1024, 2048)),
    ("w4a16_f16", (1024, 2304, 1056)), ("w4a16_bf16", (2100, 520, 544)),          # pair tiles, ragged K stage
    # M <= 64: the weight-stream kernel that expands the packed weights into tensor memory
    ("w4a16_f16", (1, 128, 64)), ("w4a16_bf16", (1, 256, 512)), ("w4a16_f16", (16, 328, 160)), ("w4a16_bf16", (40, 1000, 1056)),
    ("w4a16_bf16", (64, 4096, 4096)), ("w4a16_f16", (8, 4096, 11008)), ("w4a16_bf16", (32, 12288, 4096)),
    # 64 < M <= 128: the same kernel family with one 128-row activation tile
    ("w4a16_f16", (65, 128, 64)), ("w4a16_bf16", (100, 328, 160)), ("w4a16_f16", (128, 1000, 1056)),
    ("w4a16_bf16", (128, 4096, 4096)), ("w4a16_f16", (96, 4096, 11008)), ("w4a16_f16", (128, 12288, 4096)),
])
def test_w4a16(oracle, cuda_device, kind, shape):
    from blaze_b200 import GemmPlan
    M, N, K = shape
    act = "bf16" if kind.endswith("bf16") else "f16"
    rng_a, rng_b = np.random.default_rng(42), np.random.default_rng(123)
    enc = oracle.f32_to_bf16 if act == "bf16" else oracle.f32_to_f16
    A = enc(rng_a.standard_normal((M, K)).astype(np.float32))
    bd, bsf, gb = oracle.quantize_nvfp4((rng_b.standard_normal((N, K)) * 0.02).astype(np.float32))
    acc, alpha = oracle.gemm_w4a16(A, act, bd, bsf, gb)
    want = oracle.widen(oracle.narrow(oracle.epilogue(acc, alpha), act), act)
    C = _out_tensor(M, N, act, cuda_device)
    plan = GemmPlan(kind, M, N, K, bits16_to_torch(A, act, cuda_device), _u8(bd, cuda_device), B_sf=_u8(bsf, cuda_device), b_scale=gb, out_dtype=act)
    if M <= 128 and not (M > 64 and K >= 8192 and -(-N // 128) * 4 <= 148):
        assert plan.info()["variant"] == 3 and plan.info()["launches"] == 1    # one kernel, no expanded copy of the weights
    else:
        # the tiled kernel expands in shared memory: no 16-bit copy; a second launch only to add K splits
        assert plan.info()["launches"] == (2 if plan.info()["split_k"] > 1 else 1)
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, act), want, "w4a16 %s %s" % (kind, shape))
    plan.destroy()


@pytest.mark.parametrize("kind,shape", [("w4a16_bf16", (512, 1024, 2048)), ("w4a16_f16", (300, 520, 544)), ("w4a16_bf16", (2100, 520, 544))])
def test_w4a16_static_weights(oracle, cuda_device, kind, shape):
    """Weights declared static: expanded once at plan creation, one launch per execute; after the packed
    weights change in place, refresh_weights() brings the 16-bit copy up to date."""
    from blaze_b200 import GemmPlan
    M, N, K = shape
    act = "bf16" if kind.endswith("bf16") else "f16"
    enc = oracle.f32_to_bf16 if act == "bf16" else oracle.f32_to_f16
    A = enc(np.random.default_rng(42).standard_normal((M, K)).astype(np.float32))
    tA = bits16_to_torch(A, act, cuda_device)
    w = [oracle.quantize_nvfp4((np.random.default_rng(seed).standard_normal((N, K)) * 0.02).astype(np.float32)) for seed in (123, 321)]
    tB, tS = _u8(w[0][0], cuda_device), _u8(w[0][1], cuda_device)
    plan = GemmPlan(kind, M, N, K, tA, tB, B_sf=tS, b_scale=w[0][2], out_dtype=act, static_weights=True)
    info = plan.info()
    assert info["launches"] == (2 if info["split_k"] > 1 else 1) and info["workspace_bytes"] >= N * K * 2, info   # no expansion launch
    for i, (bd, bsf, gb) in enumerate(w):
        if i == 1:
            # same global scale is kept by the plan: re-quantise the second matrix's codes against it is not needed for
            # the check -- the oracle below uses the plan's scale with the new codes and block scales
            tB.copy_(_u8(bd, cuda_device)); tS.copy_(_u8(bsf, cuda_device))
            plan.refresh_weights()
        acc, alpha = oracle.gemm_w4a16(A, act, bd, bsf, w[0][2])
        want = oracle.widen(oracle.narrow(oracle.epilogue(acc, alpha), act), act)
        C = _out_tensor(M, N, act, cuda_device)
        _run(plan, C)
        assert_close(torch_to_f32(C, oracle, act), want, "w4a16 static weights %s %s, weights %d" % (kind, shape, i))
    plan.destroy()


@pytest.mark.parametrize("kind,shape,tiles_per_cta,mode", [
    ("w4a16_f16", (16, 1000, 1056), 3, "none"),       # 8 tiles (last ragged), request clamped to 2 per CTA; ragged K stage
    ("w4a16_f16", (16, 1000, 2080), -2, "none"),      # the same with K split over clusters of 2: 4 clusters, 9 stages as 5 + 4
    ("w4a16_bf16", (12, 896, 4096), -2, "bias_silu"), # clusters of 2, two tiles per CTA (7 tiles: 2 + 2 + 2 + 1)
    ("w4a16_bf16", (5, 1024, 512), 2, "bias_silu"),
    ("w4a16_bf16", (16, 1152, 768), 2, "none"),       # 9 tiles: 2 + 2 + 2 + 2 + 1
    ("w4a16_f16", (24, 640, 768), 7, "none"),         # M > 16: the accumulator columns hold one tile, the request is clamped
    ("w4a16_f16", (16, 1024, 512), 2, "swiglu"),
    ("w4a16_bf16", (8, 19200, 256), 0, "none"),       # 150 tiles > 148 SMs: two tiles per CTA chosen automatically
])
def test_w4a16_skinny_several_tiles_per_cta(oracle, cuda_device, monkeypatch, kind, shape, tiles_per_cta, mode):
    """The W4A16 skinny-M kernel with several consecutive weight tiles per CTA (what it does by itself
    when the tiles outnumber the SMs), forced on small shapes through BLZ_DECODE_TILES_PER_CTA."""
    from blaze_b200 import GemmPlan
    M, N, K = shape
    split = 1
    if tiles_per_cta:
        split = 2 if tiles_per_cta < 0 else 1                # negative: the same tiles per CTA with a 2-way K split
        tiles_per_cta = abs(tiles_per_cta)
        monkeypatch.setenv("BLZ_DECODE_TILES_PER_CTA", str(tiles_per_cta))
        monkeypatch.setenv("BLZ_DECODE_SPLIT", str(split))
    act = "bf16" if kind.endswith("bf16") else "f16"
    rng_a, rng_b = np.random.default_rng(42), np.random.default_rng(123)
    enc = oracle.f32_to_bf16 if act == "bf16" else oracle.f32_to_f16
    A = enc(rng_a.standard_normal((M, K)).astype(np.float32))
    bd, bsf, gb = oracle.quantize_nvfp4((rng_b.standard_normal((N, K)) * 0.02).astype(np.float32))
    acc, alpha = oracle.gemm_w4a16(A, act, bd, bsf, gb)
    kw = {}
    if mode == "swiglu":
        # rows of B read as 16 gate rows, 16 up rows, ...: outputs [M, N/2]
        g_rows = np.arange(N).reshape(N // 32, 2, 16)[:, 0].reshape(-1); u_rows = g_rows + 16
        want32 = oracle.swiglu(acc[:, g_rows], alpha, acc[:, u_rows], alpha)
        n_out = N // 2
    elif mode == "bias_silu":
        bias32 = np.random.default_rng(5).standard_normal(N).astype(np.float32)
        bias_n = oracle.widen(oracle.narrow(bias32, act), act)
        want32 = oracle.epilogue(acc, alpha, bias=bias_n, mode=mode)
        kw["bias"] = bits16_to_torch(oracle.narrow(bias32, act), act, cuda_device)
        n_out = N
    else:
        want32 = oracle.epilogue(acc, alpha)
        n_out = N
    want = oracle.widen(oracle.narrow(want32, act), act)
    C = _out_tensor(M, n_out, act, cuda_device)
    plan = GemmPlan(kind, M, N, K, bits16_to_torch(A, act, cuda_device), _u8(bd, cuda_device), B_sf=_u8(bsf, cuda_device), b_scale=gb, out_dtype=act,
                    epilogue=mode, **kw)
    info = plan.info()
    n_tiles = -(-N // 128)
    if tiles_per_cta:
        t_eff = min(tiles_per_cta, 2 if M <= 16 else 1)
        assert info["variant"] == 3 and info["split_k"] == split and info["grid"] == -(-n_tiles // t_eff) * split, info
    else:
        t_eff = 0
        assert info["variant"] == 3 and info["grid"] <= 148 and info["grid"] < n_tiles * info["split_k"], info
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, act), want, "w4a16 skinny, %d tiles per CTA, %s %s" % (t_eff, kind, shape))
    plan.destroy()


@pytest.mark.parametrize("static_weights", [False, True])
def test_w4a16_config4_sampled(oracle, cuda_device, static_weights):
    """The W4A16 prefill configuration at full size: M=4096, N=22016, K=4096, bf16 activations N(0,1), weights
    N(0,0.02) as NVFP4 -- expanded inside the kernel (default) and from a 16-bit copy made once (static weights)."""
    torch = _torch()
    from blaze_b200 import GemmPlan, quantize_nvfp4
    M, N, K = 4096, 22016, 4096
    ga = torch.Generator(device=cuda_device).manual_seed(42)
    gb = torch.Generator(device=cuda_device).manual_seed(123)
    A = torch.randn((M, K), generator=ga, device=cuda_device).to(torch.bfloat16)
    W = torch.randn((N, K), generator=gb, device=cuda_device) * 0.02
    bd, bsf, gB = quantize_nvfp4(W, tiled=False); del W
    gB = float(gB.item())
    C = _out_tensor(M, N, "bf16", cuda_device)
    plan = GemmPlan("w4a16_bf16", M, N, K, A, bd, B_sf=bsf, b_scale=gB, out_dtype="bf16", static_weights=static_weights)
    assert plan.info()["launches"] == 1
    _run(plan, C)
    rows = np.array(sorted(set(np.random.default_rng(11).integers(0, M, 22).tolist() + [0, M - 1])))
    ridx = torch.from_numpy(rows).to(cuda_device)
    a_raw = A[ridx].view(torch.int16).cpu().numpy().view(np.uint16)
    acc, alpha = oracle.gemm_w4a16(a_raw, "bf16", bd.cpu().numpy(), bsf.cpu().numpy(), gB)
    want = oracle.widen(oracle.narrow(oracle.epilogue(acc, alpha), "bf16"), "bf16")
    assert_close(torch_to_f32(C[ridx], oracle, "bf16"), want, "config 4 sampled rows")
    plan.destroy()


# ------------------------------------------------------------------- fused gate + up (SwiGLU)

def _interleave_rows16(g, u):
    """[n, w] x 2 -> [2n, w]: groups of 16 rows alternately from g and u (the layout the epilogue expects)."""
    n, w = g.shape
    return np.ascontiguousarray(np.stack([g.reshape(n // 16, 16, w), u.reshape(n // 16, 16, w)], axis=1).reshape(2 * n, w))


@pytest.mark.parametrize("kind,variant,shape", [
    ("w4a16_f16", "auto", (1, 176, 256)),            # skinny-M kernels: a single row
    ("w4a16_bf16", "auto", (100, 176, 160)),         # 128-row activation tile, ragged last weight tile
    ("w4a16_bf16", "auto", (16, 2048, 4096)),        # K split over the cluster
    ("nvfp4", "auto", (16, 400, 512)),
    ("fp8", "auto", (48, 144, 256)),
    ("bf16", "auto", (8, 144, 192)),
    ("w4a16_f16", "128x128", (24, 176, 256)),        # the tiled kernel on few rows
    ("w4a16_f16", "auto", (300, 1024, 1056)),        # ragged M and K stage
    ("w4a16_bf16", "256x256", (520, 1024, 512)),     # CTA pairs
    ("w4a16_bf16", "auto", (2100, 272, 544)),        # M > 2048: 16-bit copy of the weights first
    ("bf16", "auto", (160, 144, 192)),
    ("fp8", "auto", (160, 144, 256)),
    ("nvfp4", "256x256", (384, 400, 512)),
])
def test_swiglu_one_kernel(oracle, cuda_device, kind, variant, shape):
    """C[M, N] = silu(x Wg^T) * (x Wu^T) from ONE GEMM over the 2N interleaved weight rows, against the
    oracle's two separate products; different tensor scales for the two weights."""
    from blaze_b200 import GemmPlan, interleave_gate_up
    M, N, K = shape
    rng_a, rng_g, rng_u = np.random.default_rng(42), np.random.default_rng(123), np.random.default_rng(124)
    kw = {}
    if kind.startswith("w4a16"):
        act = "bf16" if kind.endswith("bf16") else "f16"
        enc = oracle.f32_to_bf16 if act == "bf16" else oracle.f32_to_f16
        A = enc(rng_a.standard_normal((M, K)).astype(np.float32))
        gd, gsf, gg = oracle.quantize_nvfp4((rng_g.standard_normal((N, K)) * 0.02).astype(np.float32))
        ud, usf, gu = oracle.quantize_nvfp4((rng_u.standard_normal((N, K)) * 0.05).astype(np.float32))
        acc_g, alpha_g = oracle.gemm_w4a16(A, act, gd, gsf, gg)
        acc_u, alpha_u = oracle.gemm_w4a16(A, act, ud, usf, gu)
        a_dev = bits16_to_torch(A, act, cuda_device)
        # the device helper interleaves the K-major packed rows and the row-major scales in groups of 16 rows
        b_dev = interleave_gate_up(_u8(gd, cuda_device), _u8(ud, cuda_device), 16 * K // 2)
        sf_dev = interleave_gate_up(_u8(gsf, cuda_device), _u8(usf, cuda_device), 16 * K // 16)
        assert np.array_equal(b_dev.cpu().numpy().reshape(2 * N, K // 2), _interleave_rows16(gd, ud))
        kw = dict(B_sf=sf_dev, b_scale=gg, b_scale2=gu)
        out = act
    elif kind == "bf16":
        A, G = _dense_inputs(oracle, "bf16", M, N, K, scale=0.25)
        U = oracle.f32_to_bf16((rng_u.standard_normal((N, K)) * 0.25).astype(np.float32))
        acc_g, acc_u = oracle.gemm_dense16(A, G, "bf16"), oracle.gemm_dense16(A, U, "bf16")
        alpha_g = alpha_u = 1.0
        a_dev = bits16_to_torch(A, "bf16", cuda_device)
        b_dev = bits16_to_torch(_interleave_rows16(G, U), "bf16", cuda_device)
        out = "bf16"
    elif kind == "fp8":
        qa, da, qg, dg = _fp8_inputs(oracle, M, N, K)
        xu = rng_u.uniform(-1, 1, (N, K)).astype(np.float32) * 3.0
        qu, su = oracle.quantize_fp8(xu)
        du = float(np.float32(1.0) / np.float32(su))
        acc_g = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qg)); alpha_g = float(np.float32(da) * np.float32(dg))
        acc_u = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qu)); alpha_u = float(np.float32(da) * np.float32(du))
        a_dev = _u8(qa, cuda_device)
        b_dev = _u8(_interleave_rows16(qg, qu), cuda_device)
        kw = dict(a_scale=da, b_scale=dg, b_scale2=du)
        out = "f16"
    else:
        (ad, asf, ga), (gd, gsf, gg) = _nvfp4_inputs(oracle, M, N, K)
        ud, usf, gu = oracle.quantize_nvfp4((rng_u.standard_normal((N, K)) * 0.5).astype(np.float32))
        acc_g, alpha_g = oracle.gemm_nvfp4(ad, asf, ga, gd, gsf, gg)
        acc_u, alpha_u = oracle.gemm_nvfp4(ad, asf, ga, ud, usf, gu)
        a_dev = _u8(ad, cuda_device)
        b_dev = _u8(_interleave_rows16(gd, ud), cuda_device)
        kw = dict(A_sf=_u8(asf, cuda_device), B_sf=_u8(_interleave_rows16(gsf, usf), cuda_device), a_scale=ga, b_scale=gg, b_scale2=gu)
        out = "bf16"
    want = oracle.widen(oracle.narrow(oracle.swiglu(acc_g, alpha_g, acc_u, alpha_u), out), out)
    C = _out_tensor(M, N, out, cuda_device)
    plan = GemmPlan(kind, M, 2 * N, K, a_dev, b_dev, out_dtype=out, epilogue="swiglu", variant=variant, **kw)
    info = plan.info()
    skinny = variant == "auto" and M <= (128 if kind.startswith("w4a16") else 64)
    assert (info["variant"] == 3) == skinny and (skinny or info["split_k"] == 1)
    assert info["launches"] == 1
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, out), want, "swiglu %s %s" % (kind, shape))
    plan.destroy()


def test_swiglu_blaze_layout_strided(oracle, cuda_device):
    """The mirror of Blaze's launch_fused_gate_up: weights in its [K, N/2] / [K/16, N] convention,
    fp16 in and out; also a strided output and the argument checks of the epilogue."""
    from blaze_b200 import GemmPlan, create_fused_gate_up_plan, interleave_gate_up
    from blaze_b200 import _native as nv
    M, N, K = 200, 208, 320
    rng_a, rng_g, rng_u = np.random.default_rng(42), np.random.default_rng(123), np.random.default_rng(124)
    A = oracle.f32_to_f16(rng_a.standard_normal((M, K)).astype(np.float32))
    q = [oracle.quantize_nvfp4((r.standard_normal((N, K)) * 0.03).astype(np.float32)) for r in (rng_g, rng_u)]
    acc_g, alpha_g = oracle.gemm_w4a16(A, "f16", *q[0])
    acc_u, alpha_u = oracle.gemm_w4a16(A, "f16", *q[1])
    want = oracle.widen(oracle.narrow(oracle.swiglu(acc_g, alpha_g, acc_u, alpha_u), "f16"), "f16")

    def blaze_tensor(bd, bsf, g):
        nib = np.empty((N, K), np.uint8); nib[:, 0::2] = bd & 15; nib[:, 1::2] = bd >> 4
        nib_kn = np.ascontiguousarray(nib.T)
        return {"data": _u8(nib_kn[:, 0::2] | (nib_kn[:, 1::2] << 4), cuda_device), "block_scales": _u8(np.ascontiguousarray(bsf.T), cuda_device), "tensor_scale": g}

    Wg, Wu = blaze_tensor(*q[0]), blaze_tensor(*q[1])
    a_dev = bits16_to_torch(A, "f16", cuda_device)
    C = _out_tensor(M, N, "f16", cuda_device)
    plan = create_fused_gate_up_plan(a_dev, Wg, Wu, M, N, K)
    assert plan.info()["launches"] == 1
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, "f16"), want, "fused gate+up, Blaze layout")
    plan.destroy()
    # strided output: the columns beyond N keep their fill value
    ldc = N + 24
    data = interleave_gate_up(Wg["data"], Wu["data"], 8)
    sf = interleave_gate_up(Wg["block_scales"], Wu["block_scales"], 16)
    C2 = _out_tensor(M, N, "f16", cuda_device, ldc=ldc)
    plan = GemmPlan("w4a16_f16", M, 2 * N, K, a_dev, data, B_sf=sf, b_scale=q[0][2], b_scale2=q[1][2], out_dtype="f16", epilogue="swiglu",
                    b_layout="nmajor", ldc=ldc)
    _run(plan, C2)
    assert_close(torch_to_f32(C2[:, :N].contiguous(), oracle, "f16"), want, "fused gate+up, strided C")
    assert bool((C2[:, N:] == -7.0).all())
    plan.destroy()
    for bad in (dict(N=2 * N + 16), dict(ldc=N - 8)):
        args = dict(N=2 * N, variant="auto", ldc=0); args.update(bad)
        with pytest.raises(nv.BlazeError):
            GemmPlan("w4a16_f16", M, args["N"], K, a_dev, data, B_sf=sf, b_scale=1.0, out_dtype="f16", epilogue="swiglu", b_layout="nmajor",
                     variant=args["variant"], ldc=args["ldc"])


# ---------------------------------------------------------------------------------- epilogues

@pytest.mark.parametrize("mode", ["bias", "silu", "bias_silu", "residual"])
@pytest.mark.parametrize("kind,out_dtype", [("fp8", "f16"), ("nvfp4", "bf16"), ("bf16", "f32")])
@pytest.mark.parametrize("M", [160, 24])           # tiled kernel / skinny-M kernel
def test_epilogues(oracle, cuda_device, mode, kind, out_dtype, M):
    from blaze_b200 import GemmPlan
    torch = _torch()
    N, K = 264, 256
    rng = np.random.default_rng(77)
    bias32 = rng.standard_normal(N).astype(np.float32)
    res32 = rng.standard_normal((M, N)).astype(np.float32)
    bias_n = oracle.widen(oracle.narrow(bias32, out_dtype), out_dtype)
    res_n = oracle.widen(oracle.narrow(res32, out_dtype), out_dtype)

    def dev(x32):
        if out_dtype == "f32":
            return torch.from_numpy(x32).to(cuda_device)
        return bits16_to_torch(oracle.narrow(x32, out_dtype), out_dtype, cuda_device)

    kw = {}
    if kind == "fp8":
        qa, da, qb, db = _fp8_inputs(oracle, M, N, K)
        acc = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qb)); alpha = float(np.float32(da) * np.float32(db))
        args = (_u8(qa, cuda_device), _u8(qb, cuda_device)); kw = dict(a_scale=da, b_scale=db)
    elif kind == "nvfp4":
        (ad, asf, ga), (bd, bsf, gb) = _nvfp4_inputs(oracle, M, N, K)
        acc, alpha = oracle.gemm_nvfp4(ad, asf, ga, bd, bsf, gb)
        args = (_u8(ad, cuda_device), _u8(bd, cuda_device)); kw = dict(A_sf=_u8(asf, cuda_device), B_sf=_u8(bsf, cuda_device), a_scale=ga, b_scale=gb)
    else:
        A, Bt = _dense_inputs(oracle, "bf16", M, N, K, scale=0.25)
        acc = oracle.gemm_dense16(A, Bt, "bf16"); alpha = 1.0
        args = (bits16_to_torch(A, "bf16", cuda_device), bits16_to_torch(Bt, "bf16", cuda_device))
    want32 = oracle.epilogue(acc, alpha, bias=bias_n if "bias" in mode else None, residual=res_n if mode == "residual" else None, mode=mode)
    want = oracle.widen(oracle.narrow(want32, out_dtype), out_dtype)
    C = _out_tensor(M, N, out_dtype, cuda_device)
    plan = GemmPlan(kind, M, N, K, *args, out_dtype=out_dtype, epilogue=mode, bias=dev(bias32) if "bias" in mode else None,
                    residual=dev(res32) if mode == "residual" else None, **kw)
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, out_dtype), want, "epilogue %s %s" % (mode, kind))
    plan.destroy()


@pytest.mark.parametrize("mode", ["bias", "silu", "bias_silu", "residual"])
@pytest.mark.parametrize("M", [24, 100])            # 64-row and 128-row activation tiles
def test_epilogues_w4a16_skinny(oracle, cuda_device, mode, M):
    """The kernels that expand the packed weights into tensor memory share the skinny-M epilogue;
    M = 100 goes through its chunked form, K = 1056 through a ragged last load stage."""
    from blaze_b200 import GemmPlan
    N, K, act = 392, 1056, "bf16"
    rng = np.random.default_rng(78)
    A = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    bd, bsf, gb = oracle.quantize_nvfp4((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    bias_n = oracle.widen(oracle.narrow(rng.standard_normal(N).astype(np.float32), act), act)
    res_n = oracle.widen(oracle.narrow(rng.standard_normal((M, N)).astype(np.float32), act), act)
    acc, alpha = oracle.gemm_w4a16(A, act, bd, bsf, gb)
    want32 = oracle.epilogue(acc, alpha, bias=bias_n if "bias" in mode else None, residual=res_n if mode == "residual" else None, mode=mode)
    want = oracle.widen(oracle.narrow(want32, act), act)
    C = _out_tensor(M, N, act, cuda_device)
    plan = GemmPlan("w4a16_bf16", M, N, K, bits16_to_torch(A, act, cuda_device), _u8(bd, cuda_device), B_sf=_u8(bsf, cuda_device), b_scale=gb,
                    out_dtype=act, epilogue=mode,
                    bias=bits16_to_torch(oracle.narrow(bias_n, act), act, cuda_device) if "bias" in mode else None,
                    residual=bits16_to_torch(oracle.narrow(res_n, act), act, cuda_device) if mode == "residual" else None)
    assert plan.info()["variant"] == 3
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, act), want, "w4a16 skinny epilogue %s M=%d" % (mode, M))
    plan.destroy()


def test_strided_output_and_fp16_saturation(oracle, cuda_device):
    """ldc > N leaves the padding untouched; fp16 stores clamp to +-65504 (no infinities)."""
    from blaze_b200 import GemmPlan
    M, N, K, ldc = 130, 136, 128, 160
    qa, da, qb, db = _fp8_inputs(oracle, M, N, K)
    C = _out_tensor(M, N, "f16", cuda_device, ldc=ldc)
    plan = GemmPlan("fp8", M, N, K, _u8(qa, cuda_device), _u8(qb, cuda_device), a_scale=1.0, b_scale=1.0, out_dtype="f16", ldc=ldc)
    _run(plan, C)
    acc = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qb))
    want = oracle.widen(oracle.narrow(acc, "f16"), "f16")
    got = torch_to_f32(C, oracle, "f16")
    assert np.abs(want).max() == 65504.0                       # the raw E4M3 product overflows fp16 here
    assert_close(got[:, :N], want, "fp16 saturating store")
    assert np.all(got[:, N:] == -7.0)
    plan.destroy()


def test_run_to_run_bit_identical(oracle, cuda_device):
    from blaze_b200 import GemmPlan
    torch = _torch()
    M, N, K = 1024, 2048, 2048
    (ad, asf, ga), (bd, bsf, gb) = _nvfp4_inputs(oracle, M, N, K)
    plan = GemmPlan("nvfp4", M, N, K, _u8(ad, cuda_device), _u8(bd, cuda_device), A_sf=_u8(asf, cuda_device), B_sf=_u8(bsf, cuda_device),
                    a_scale=ga, b_scale=gb, out_dtype="bf16")
    outs = []
    for _ in range(3):
        C = _out_tensor(M, N, "bf16", cuda_device)
        _run(plan, C)
        outs.append(C)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    plan.destroy()


def test_set_a_rebinds_activations(oracle, cuda_device):
    from blaze_b200 import GemmPlan, tile_scales
    M, N, K = 16, 512, 1024
    qa, qb = _nvfp4_inputs(oracle, M, N, K)
    (ad, asf, ga), (bd, bsf, gb) = qa, qb
    rng = np.random.default_rng(1234)
    ad2, asf2, ga2 = oracle.quantize_nvfp4(rng.standard_normal((M, K)).astype(np.float32))
    t_asf = tile_scales(_u8(asf, cuda_device), M, K)
    t_asf2 = tile_scales(_u8(asf2, cuda_device), M, K)
    assert np.array_equal(t_asf.cpu().numpy(), oracle.tile_sf(asf, 2, (K // 64 + 3) // 4 * 4))
    C = _out_tensor(M, N, "bf16", cuda_device)
    plan = GemmPlan("nvfp4", M, N, K, _u8(ad, cuda_device), _u8(bd, cuda_device), A_sf=t_asf, B_sf=_u8(bsf, cuda_device),
                    a_scale=ga, b_scale=gb, out_dtype="bf16", a_sf_layout="tiled")
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, "bf16"), _nvfp4_ref(oracle, qa, qb), "before set_a")
    plan.set_a(_u8(ad2, cuda_device), t_asf2, ga2)
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, "bf16"), _nvfp4_ref(oracle, (ad2, asf2, ga2), qb), "after set_a")
    plan.destroy()


@pytest.mark.parametrize("kind,M", [("w4a16_bf16", 24), ("w4a16_f16", 100), ("fp8", 48), ("bf16", 8), ("bf16", 300)])
def test_set_a_other_kinds(oracle, cuda_device, kind, M):
    """Rebinding the activations of a plan (decode loops reuse one plan per weight matrix): the
    skinny-M kernels of every kind and the tiled kernel."""
    from blaze_b200 import GemmPlan
    N, K = 392, 1056 if kind != "fp8" else 1040
    rng = np.random.default_rng(4321)

    def make_a(seed):
        x = np.random.default_rng(seed).standard_normal((M, K)).astype(np.float32)
        if kind == "fp8":
            q, s = oracle.quantize_fp8(x)
            return q, float(np.float32(1.0) / np.float32(s))
        enc = oracle.f32_to_f16 if kind.endswith("f16") and not kind.endswith("bf16") else oracle.f32_to_bf16
        return enc(x), 1.0

    act = "f16" if kind == "w4a16_f16" else "bf16"
    if kind.startswith("w4a16"):
        bd, bsf, gb = oracle.quantize_nvfp4((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
        ref = lambda a, sa: oracle.epilogue(*oracle.gemm_w4a16(a, act, bd, bsf, gb))
        to_dev = lambda a: bits16_to_torch(a, act, cuda_device)
        b_args, kw = (_u8(bd, cuda_device),), dict(B_sf=_u8(bsf, cuda_device), b_scale=gb)
    elif kind == "fp8":
        qb, sb = oracle.quantize_fp8(rng.uniform(-1, 1, (N, K)).astype(np.float32))
        db = float(np.float32(1.0) / np.float32(sb))
        ref = lambda a, sa: oracle.epilogue(oracle.gemm_f32(oracle.e4m3_to_f32(a), oracle.e4m3_to_f32(qb)), float(np.float32(sa) * np.float32(db)))
        to_dev = lambda a: _u8(a, cuda_device)
        b_args, kw = (_u8(qb, cuda_device),), dict(b_scale=db)
    else:
        Bt = oracle.f32_to_bf16(rng.standard_normal((N, K)).astype(np.float32))
        ref = lambda a, sa: oracle.gemm_dense16(a, Bt, "bf16")
        to_dev = lambda a: bits16_to_torch(a, "bf16", cuda_device)
        b_args, kw = (bits16_to_torch(Bt, "bf16", cuda_device),), {}
    (a1, s1), (a2, s2) = make_a(1), make_a(2)
    C = _out_tensor(M, N, act, cuda_device)
    if kind == "fp8":
        kw["a_scale"] = s1
    plan = GemmPlan(kind, M, N, K, to_dev(a1), *b_args, out_dtype=act, **kw)
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, act), oracle.widen(oracle.narrow(ref(a1, s1), act), act), "%s M=%d before set_a" % (kind, M))
    d2 = to_dev(a2)
    plan.set_a(d2, None, s2 if kind == "fp8" else 0.0)
    _run(plan, C)
    assert_close(torch_to_f32(C, oracle, act), oracle.widen(oracle.narrow(ref(a2, s2), act), act), "%s M=%d after set_a" % (kind, M))
    plan.destroy()


@pytest.mark.parametrize("exchange", ["none", "nccl", "peer_stores"])
def test_sharded_plan_one_rank(oracle, cuda_device, exchange):
    """The C-level sharded plan with a world of one (the driver's single-GPU box): shard = everything, every
    exchange degenerates to the local result; two or more ranks are covered by the two-GPU test."""
    from blaze_b200 import sharded
    torch = _torch()
    M, N, K = 512, 1024, 512
    qa, da, qb, db = _fp8_inputs(oracle, M, N, K)
    acc = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qb))
    want = oracle.widen(oracle.narrow(oracle.epilogue(acc, float(np.float32(da) * np.float32(db))), "bf16"), "bf16")
    sp = sharded.ShardedPlan("fp8", M, N, K, _u8(qa, cuda_device), _u8(qb, cuda_device), exchange=exchange, a_scale=da, b_scale=db, out_dtype="bf16")
    assert (sp.col_lo, sp.col_hi) == (0, N)
    if exchange == "peer_stores":
        sp.output.fill_(-7.0)
        sp.execute(); sp.check()
        got = sp.output.clone()
    else:
        got = _out_tensor(M, N, "bf16", cuda_device)
        sp.execute(got); sp.check()
    assert_close(torch_to_f32(got, oracle, "bf16"), want, "sharded plan, one rank, exchange %s" % exchange)
    sp.destroy()


# ----------------------------------------------------------- the split tail of the tile schedule

@pytest.mark.parametrize("kind,variant,shape,mode,out_dtype", [
    ("nvfp4", "256x256", (2304, 2304, 4096), "none", "bf16"),       # 81 tiles on 74 pairs: 7 tail tiles, each cut along K
    ("nvfp4", "128x128", (1300, 2000, 2048), "none", "bf16"),       # ragged M and N; 176 tiles on 148 CTAs
    ("fp8", "128x128", (1280, 2048, 6144), "bias_silu", "f16"),     # the reduce kernel applies bias and SiLU
    ("fp8", "256x256", (2304, 2304, 2048), "residual", "bf16"),
    ("bf16", "256x256", (2300, 2300, 1096), "none", "f32"),         # ragged in M, N and the last K stage
    ("f16", "256x256", (512, 2048, 4096), "none", "bf16"),          # 16 tiles for 74 pairs: every tile is cut (four units each)
    ("fp8", "256x256", (500, 1000, 11008), "bias", "bf16"),         # 8 ragged tiles, nine units each
    ("nvfp4", "256x256", (8192, 3584, 2048), "none", "bf16"),       # 448 tiles = 6 waves + 4 tiles of 8 units (one rank's shard shape, shorter K)
])
def test_tail_split(oracle, cuda_device, kind, variant, shape, mode, out_dtype):
    """When the last wave of the schedule is at most half full, its tiles are cut along K; the units of a tile
    exchange fp32 partial sums inside the launch and each finishes a slice of the tile in unit order: same result
    as the oracle, and the same bits run to run."""
    from blaze_b200 import GemmPlan
    torch = _torch()
    M, N, K = shape
    rng = np.random.default_rng(91)
    bias_n = oracle.widen(oracle.narrow(rng.standard_normal(N).astype(np.float32), out_dtype), out_dtype)
    res_n = oracle.widen(oracle.narrow(rng.standard_normal((M, N)).astype(np.float32), out_dtype), out_dtype)
    if kind == "nvfp4":
        qa, qb = _nvfp4_inputs(oracle, M, N, K)
        (ad, asf, ga), (bd, bsf, gb) = qa, qb
        acc, alpha = oracle.gemm_nvfp4(ad, asf, ga, bd, bsf, gb)
        args = (_u8(ad, cuda_device), _u8(bd, cuda_device)); kw = dict(A_sf=_u8(asf, cuda_device), B_sf=_u8(bsf, cuda_device), a_scale=ga, b_scale=gb)
    elif kind == "fp8":
        qa, da, qb, db = _fp8_inputs(oracle, M, N, K)
        acc = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qb)); alpha = float(np.float32(da) * np.float32(db))
        args = (_u8(qa, cuda_device), _u8(qb, cuda_device)); kw = dict(a_scale=da, b_scale=db)
    else:
        A, Bt = _dense_inputs(oracle, kind, M, N, K, scale=0.25)
        acc = oracle.gemm_dense16(A, Bt, kind); alpha = 1.0
        args = (bits16_to_torch(A, kind, cuda_device), bits16_to_torch(Bt, kind, cuda_device)); kw = {}
    want32 = oracle.epilogue(acc, alpha, bias=bias_n if "bias" in mode else None, residual=res_n if mode == "residual" else None, mode=mode)
    want = oracle.widen(oracle.narrow(want32, out_dtype), out_dtype)

    def dev(x32):
        if out_dtype == "f32":
            return torch.from_numpy(np.ascontiguousarray(x32, np.float32)).to(cuda_device)
        return bits16_to_torch(oracle.narrow(x32, out_dtype), out_dtype, cuda_device)
    plan = GemmPlan(kind, M, N, K, *args, out_dtype=out_dtype, variant=variant, epilogue=mode, bias=dev(bias_n) if "bias" in mode else None,
                    residual=dev(res_n) if mode == "residual" else None, tail_split=True, **kw)
    info = plan.info()
    assert info["tail_tiles"] > 0 and info["tail_split"] >= 2 and info["launches"] == 1, info
    outs = []
    for _ in range(3):
        C = _out_tensor(M, N, out_dtype, cuda_device)
        _run(plan, C)
        outs.append(C)
    assert_close(torch_to_f32(outs[0], oracle, out_dtype), want, "tail split %s %s %s %s" % (kind, variant, shape, info))
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    plan.destroy()


# ------------------------------------------------------------ dynamic tile scheduler (cluster launch control)

@pytest.mark.parametrize("kind,variant,shape", [
    ("nvfp4", "256x256", (2048, 2304, 1024)),     # 72 tiles over the pairs that are resident
    ("nvfp4", "256x256", (4096, 8192, 512)),      # 512 tiles of 256x256 on 74 pairs: most tiles are taken over by running clusters
    ("nvfp4", "128x128", (1100, 4000, 416)),      # ragged M, N and K stage; 288 tiles of 128x128
    ("nvfp4", "256x384", (1024, 1536, 512)),
    ("fp8", "256x256", (4096, 4096, 256)),
    ("fp8", "128x128", (300, 5000, 144)),
    ("bf16", "256x256", (3000, 2304, 136)),
    ("f16", "128x128", (2048, 2176, 64)),
    ("fp8", "128x128", (128, 512, 8192)),         # with the tiled kernel's K split (tiles = splits x tiles)
])
def test_clc_scheduler(oracle, cuda_device, kind, variant, shape):
    """Every tile the hardware hands out is computed exactly once: the result equals the oracle and, bit for bit,
    what the static persistent schedule gives.  Counterpart of the scheduler Blaze sketches in
    include/gemm/tmem_utils.cuh:251-305."""
    from blaze_b200 import GemmPlan
    torch = _torch()
    M, N, K = shape
    if kind == "nvfp4":
        qa, qb = _nvfp4_inputs(oracle, M, N, K)
        want = _nvfp4_ref(oracle, qa, qb)
        (ad, asf, ga), (bd, bsf, gb) = qa, qb
        args = (_u8(ad, cuda_device), _u8(bd, cuda_device))
        kw = dict(A_sf=_u8(asf, cuda_device), B_sf=_u8(bsf, cuda_device), a_scale=ga, b_scale=gb)
    elif kind == "fp8":
        qa, da, qb, db = _fp8_inputs(oracle, M, N, K)
        acc = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qb))
        want = oracle.widen(oracle.narrow(oracle.epilogue(acc, float(np.float32(da) * np.float32(db))), "bf16"), "bf16")
        args = (_u8(qa, cuda_device), _u8(qb, cuda_device))
        kw = dict(a_scale=da, b_scale=db)
    else:
        A, Bt = _dense_inputs(oracle, kind, M, N, K)
        want = oracle.widen(oracle.narrow(oracle.gemm_dense16(A, Bt, kind), "bf16"), "bf16")
        args = (bits16_to_torch(A, kind, cuda_device), bits16_to_torch(Bt, kind, cuda_device))
        kw = {}
    outs = {}
    for sched in ("clc", "static"):
        C = _out_tensor(M, N, "bf16", cuda_device)
        plan = GemmPlan(kind, M, N, K, *args, out_dtype="bf16", variant=variant, scheduler=sched, **kw)
        info = plan.info()
        assert info["scheduler"] == (1 if sched == "clc" else 0), info
        assert info["tail_tiles"] == 0, info                  # whole tiles under both schedules: the sums are formed in the same order
        for _ in range(2):                                     # twice: the launch queue is consumed anew by every launch
            C.fill_(-7.0)
            _run(plan, C)
        outs[sched] = C
        if sched == "clc":
            assert_close(torch_to_f32(C, oracle, "bf16"), want, "clc %s %s %s %s" % (kind, variant, shape, info))
        plan.destroy()
    assert torch.equal(outs["clc"], outs["static"])


@pytest.mark.parametrize("kind,shape,mode", [
    ("bf16", (128, 512, 8192), "none"), ("bf16", (200, 300, 4104), "bias_silu"), ("fp8", (100, 384, 8192), "residual"),
    ("nvfp4", (128, 512, 16384), "none"), ("nvfp4", (300, 264, 8224), "bias"), ("w4a16_f16", (200, 384, 4096), "none"),
    ("w4a16_bf16", (130, 520, 4128), "residual"),
])
def test_tiled_split_k(oracle, cuda_device, kind, shape, mode):
    """Few 128x128 tiles and a long K: the tiled kernel splits K over several CTAs per tile (fp32
    partial sums in a scratch matrix, summed in split order by a second kernel that also applies
    the epilogue); ragged M / N / K, every kind."""
    from blaze_b200 import GemmPlan
    M, N, K = shape
    rng = np.random.default_rng(99)
    out = "f16" if kind == "w4a16_f16" else "bf16"
    kw = {}
    if kind == "bf16":
        A, Bt = _dense_inputs(oracle, "bf16", M, N, K, scale=0.25)
        acc, alpha = oracle.gemm_dense16(A, Bt, "bf16"), 1.0
        args = (bits16_to_torch(A, "bf16", cuda_device), bits16_to_torch(Bt, "bf16", cuda_device))
    elif kind == "fp8":
        qa, da, qb, db = _fp8_inputs(oracle, M, N, K)
        acc, alpha = oracle.gemm_f32(oracle.e4m3_to_f32(qa), oracle.e4m3_to_f32(qb)), float(np.float32(da) * np.float32(db))
        args = (_u8(qa, cuda_device), _u8(qb, cuda_device)); kw = dict(a_scale=da, b_scale=db)
    elif kind == "nvfp4":
        (ad, asf, ga), (bd, bsf, gb) = _nvfp4_inputs(oracle, M, N, K)
        acc, alpha = oracle.gemm_nvfp4(ad, asf, ga, bd, bsf, gb)
        args = (_u8(ad, cuda_device), _u8(bd, cuda_device)); kw = dict(A_sf=_u8(asf, cuda_device), B_sf=_u8(bsf, cuda_device), a_scale=ga, b_scale=gb)
    else:
        enc = oracle.f32_to_f16 if out == "f16" else oracle.f32_to_bf16
        A = enc(rng.standard_normal((M, K)).astype(np.float32))
        bd, bsf, gb = oracle.quantize_nvfp4((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
        acc, alpha = oracle.gemm_w4a16(A, out, bd, bsf, gb)
        args = (bits16_to_torch(A, out, cuda_device), _u8(bd, cuda_device)); kw = dict(B_sf=_u8(bsf, cuda_device), b_scale=gb)
    bias_n = oracle.widen(oracle.narrow(rng.standard_normal(N).astype(np.float32), out), out)
    res_n = oracle.widen(oracle.narrow(rng.standard_normal((M, N)).astype(np.float32), out), out)
    want32 = oracle.epilogue(acc, alpha, bias=bias_n if "bias" in mode else None, residual=res_n if mode == "residual" else None, mode=mode)
    want = oracle.widen(oracle.narrow(want32, out), out)
    C = _out_tensor(M, N, out, cuda_device)
    plan = GemmPlan(kind, M, N, K, *args, out_dtype=out, epilogue=mode, variant="128x128",
                    bias=bits16_to_torch(oracle.narrow(bias_n, out), out, cuda_device) if "bias" in mode else None,
                    residual=bits16_to_torch(oracle.narrow(res_n, out), out, cuda_device) if mode == "residual" else None, **kw)
    assert plan.info()["split_k"] > 1, plan.info()
    _run(plan, C)
    first = C.clone()
    assert_close(torch_to_f32(C, oracle, out), want, "tiled split-K %s %s %s %s" % (kind, shape, mode, plan.info()))
    _run(plan, C)
    assert _torch().equal(first, C), "split-K result changed between two runs"
    plan.destroy()


# ------------------------------------------------------------------------ byte-level kernels

def test_quantizers_bit_exact(oracle, cuda_device):
    torch = _torch()
    from blaze_b200 import quantize_fp8, quantize_nvfp4
    rng = np.random.default_rng(2024)
    for (rows, K, dt) in [(64, 256, torch.float32), (200, 1040, torch.float32), (33, 4096, torch.bfloat16), (16, 160, torch.float16)]:
        x = torch.from_numpy(rng.standard_normal((rows, K)).astype(np.float32)).to(cuda_device).to(dt)
        x[1, 16:32] = 0                                         # an all-zero block
        x32 = x.float().cpu().numpy()
        q, sc = quantize_fp8(x)
        q_ref, s_ref = oracle.quantize_fp8(x32)
        assert np.float32(sc[0].item()) == np.float32(s_ref)
        assert np.array_equal(q.cpu().numpy(), q_ref)
        d, sf, g = quantize_nvfp4(x)
        d_ref, sf_ref, g_ref = oracle.quantize_nvfp4(x32)
        assert np.float32(g.item()) == np.float32(g_ref)
        assert np.array_equal(sf.cpu().numpy(), sf_ref), "block scales differ"
        assert np.array_equal(d.cpu().numpy(), d_ref), "E2M1 codes differ"
        d2, sft, _ = quantize_nvfp4(x, tiled=True)
        assert np.array_equal(d2.cpu().numpy(), d_ref)
        ka = ((K + 63) // 64 + 3) // 4 * 4
        rb = ((rows + 127) // 128 + 1) // 2 * 2
        assert np.array_equal(sft.cpu().numpy(), oracle.tile_sf(sf_ref, rb, ka))


# ------------------------------------------------------------------ failure detection

def test_lost_arrival_becomes_an_error_word(cuda_device):
    """A wait nobody completes runs out after its limit (2 ms here) and the kernel reports it through
    its status word; the context stays usable.  Nothing faults, traps or hangs."""
    torch = _torch()
    from blaze_b200 import _native as nv
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    waited = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    L = nv.lib()
    assert L.blz_wait_probe(2_000_000, status.data_ptr(), waited.data_ptr(), torch.cuda.current_stream().cuda_stream) == nv.OK
    torch.cuda.synchronize()
    assert int(status.item()) != 0
    assert 2_000_000 <= int(waited.item()) < 50_000_000
    assert L.blz_wait_probe(0, status.data_ptr(), None, None) == nv.ERR_INVALID_ARGUMENT
    # the device still works
    assert float((torch.ones(8, device=cuda_device) * 2).sum().item()) == 16.0


# ------------------------------------------------------------- Blaze's own test program

def test_blaze_test_program_builds_and_passes(cuda_device):
    """Blaze's tests/test_gemm.cu, compiled unchanged against this library's include/gemm headers
    (oracle/build_oracle.py builds it where the reference tree is present)."""
    exe = os.path.join(ROOT, "oracle", "_ref", "test_gemm")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/test_gemm not built (reference tree absent at build time)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=900)
    tail = "\n".join((r.stdout + r.stderr).splitlines()[-40:])
    assert r.returncode == 0, tail
    assert "FAIL" not in r.stdout, tail
