"""CPU tests of the oracle: golden vectors, the reference's known answers, format pins."""
import hashlib
import os
import shutil
import subprocess

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_known_bytes(oracle):
    g = np.load(os.path.join(GOLDEN, "known_bytes.npz"))
    assert np.array_equal(oracle.e4m3_to_f32(g["e4m3_codes"]), g["e4m3_values"])
    assert np.array_equal(oracle.e2m1_to_f32(g["e2m1_codes"]), g["e2m1_values"])
    assert np.array_equal(oracle.f32_to_e4m3(g["e4m3_values"]), g["e4m3_codes"])
    assert np.array_equal(oracle.f32_to_e2m1(g["e2m1_values"]), g["e2m1_codes"])


def test_formats_against_cuda_host_conversions():
    """oracle/pin_formats: every fp16/bf16/E4M3/E2M1 code and millions of encodes vs CUDA's headers."""
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("nvcc not available")
    from oracle import build_oracle
    exe = build_oracle.build_pin_formats()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 mismatches" in r.stdout


def test_golden_small_bit_exact(oracle):
    g = np.load(os.path.join(GOLDEN, "ref_gemm_cpu_fp16_48x80x96.npz"))
    A, B, C = g["A"], g["B"], g["C"]
    got_kn = oracle.gemm_f32_bkn(oracle.f16_to_f32(A), oracle.f16_to_f32(B))
    got_kmajor = oracle.gemm_f32(oracle.f16_to_f32(A), np.ascontiguousarray(oracle.f16_to_f32(B).T), nthreads=3)
    assert np.array_equal(got_kn.view(np.uint32), C.view(np.uint32))
    assert np.array_equal(got_kmajor.view(np.uint32), C.view(np.uint32))


def test_golden_256_seeded(oracle):
    """The 256^3 fp16 configuration: operands from the seeded fill (42 / 123), result digests from the reference."""
    g = np.load(os.path.join(GOLDEN, "ref_gemm_cpu_fp16_256.npz"))
    M = N = K = 256
    A = oracle.f32_to_f16(oracle.fill_uniform_rand(M * K, 42)).reshape(M, K)
    B = oracle.f32_to_f16(oracle.fill_uniform_rand(K * N, 123)).reshape(K, N)
    assert np.array_equal(A.reshape(-1)[:64], g["A_head"]) and sha(A) == str(g["sha_A"])
    assert np.array_equal(B.reshape(-1)[:64], g["B_head"]) and sha(B) == str(g["sha_B"])
    C = oracle.gemm_f32(oracle.f16_to_f32(A), np.ascontiguousarray(oracle.f16_to_f32(B).T))
    assert np.array_equal(C[g["rows"]].view(np.uint32), g["C_rows"].view(np.uint32))
    assert sha(C) == str(g["sha_C"])


def test_against_compiled_reference(oracle):
    """Shapes of Blaze's tests/test_gemm_naive.cu:153-162 (the small ones), bit for bit."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (reference tree absent)")
    for (M, N, K) in [(1, 256, 128), (32, 128, 256), (128, 128, 128), (100, 72, 56)]:
        A = oracle.ref_init_random_fp16(M * K, 42).reshape(M, K)
        B = oracle.ref_init_random_fp16(K * N, 123).reshape(K, N)
        want = oracle.ref_gemm_cpu_fp16(A, B)
        got = oracle.gemm_f32(oracle.f16_to_f32(A), np.ascontiguousarray(oracle.f16_to_f32(B).T), nthreads=4)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (M, N, K)


def test_blockscaled_known_answer(oracle):
    """tests/test_gemm.cu:338-389: data 0x22 (1.0, 1.0), scales 0x38 (1.0), tensor scale 1 => C == K."""
    M, N, K = 5, 24, 256
    a_data = np.full((M, K // 2), 0x22, np.uint8); a_sf = np.full((M, K // 16), 0x38, np.uint8)
    b_data = np.full((N, K // 2), 0x22, np.uint8); b_sf = np.full((N, K // 16), 0x38, np.uint8)
    acc, alpha = oracle.gemm_nvfp4(a_data, a_sf, 1.0, b_data, b_sf, 1.0)
    assert alpha == 1.0 and np.all(acc == K)


def test_fp8_all_ones_tile(oracle):
    """tests/test_sm100_primitives.cu:446-457: all-ones E4M3 128x128x64 tile => 64."""
    q = np.full((128, 64), 0x38, np.uint8)
    acc, _ = oracle.gemm_fp8(q, q, 1.0, 1.0)
    assert np.all(acc == 64.0)


def test_nibble_order_and_scale_blocks(oracle):
    data = np.zeros((1, 16), np.uint8); sf = np.array([[0x38, 0x3C]], np.uint8)   # K = 32
    data[0, 0] = 0x52            # k=0 -> 0x2 (1.0), k=1 -> 0x5 (3.0)
    data[0, 8] = 0x0A            # k=16 -> 0xA (-1.0) scaled by 1.5
    x = oracle.dequant_nvfp4_noglobal(data, sf)
    assert x[0, 0] == 1.0 and x[0, 1] == 3.0 and x[0, 16] == -1.5 and x[0, 17] == 0.0


def test_quantizers(oracle):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((48, 256)).astype(np.float32)
    q, s = oracle.quantize_fp8(x)
    assert np.float32(s) == np.float32(448.0) / np.abs(x).max()
    xd = oracle.e4m3_to_f32(q) / np.float32(s)
    assert np.abs(xd - x).max() <= np.abs(x).max() / 16 + 1e-6        # 3 mantissa bits
    data, sf, g = oracle.quantize_nvfp4(x)
    assert np.float32(g) == np.abs(x).max() / np.float32(2688.0)
    xh = oracle.dequant_nvfp4_noglobal(data, sf) * np.float32(g)
    assert np.abs(xh - x).mean() / np.abs(x).mean() < 0.12
    # idempotence: quantising the dequantised matrix with the same global scale reproduces the codes
    d2, sf2, _ = oracle.quantize_nvfp4(xh, g)
    assert np.array_equal(sf2, sf) and np.array_equal(d2, data)
    # zero block -> zero scale and zero codes
    x[3, 32:48] = 0
    data, sf, _ = oracle.quantize_nvfp4(x)
    assert sf[3, 2] == 0 and not data[3, 16:24].any()


def test_tiled_scale_layout(oracle):
    rows, kb = 200, 10
    sf = (np.arange(rows * kb) % 251).astype(np.uint8).reshape(rows, kb)
    rb, ka = 2, 4
    t = oracle.tile_sf(sf, rb, ka)
    assert t.size == rb * ka * 512
    for (r, b) in [(0, 0), (31, 3), (32, 0), (127, 9), (128, 4), (199, 9)]:
        off = ((r // 128) * ka + b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4
        assert t[off] == sf[r, b]
    assert int((t != 0).sum()) == int((sf != 0).sum())


def test_epilogue_and_narrow(oracle):
    c = np.array([[1.0, -2.0, 70000.0, 0.5]], np.float32)
    out = oracle.epilogue(c, alpha=2.0, bias=np.array([1, 1, 1, 1], np.float32), mode="bias_silu")
    v = np.float32(2.0) * c[0] + 1
    np.testing.assert_allclose(out[0], v / (1 + np.exp(-v)), rtol=1e-6)
    h = oracle.widen(oracle.narrow(np.array([70000.0, -1e9, 1.0], np.float32), "f16"), "f16")
    assert h.tolist() == [65504.0, -65504.0, 1.0]                      # saturating fp16 store
    assert oracle.widen(oracle.narrow(np.array([1.00390625], np.float32), "bf16"), "bf16")[0] == 1.0   # ties to even


def test_swiglu(oracle):
    g = np.array([[1.0, -3.0, 0.0, 8.0]], np.float32)
    u = np.array([[2.0, 0.5, 7.0, -1.0]], np.float32)
    out = oracle.swiglu(g, 0.5, u, 2.0)
    x = np.float32(0.5) * g[0]
    np.testing.assert_allclose(out[0], x / (1 + np.exp(-x)) * (2.0 * u[0]), rtol=1e-6)
    assert out[0, 2] == 0.0
