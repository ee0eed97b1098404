"""numpy front end of the CPU oracle (blaze_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke entry and the bench's CPU-baseline / reference leg may import this module;
the product package never does.  Every array in and out is a C-contiguous numpy array.

Layout conventions (the same as the CUDA library's C-ABI):
  A  : [M, K] row-major ("K-major")
  Bt : [N, K] row-major, i.e. B stored K-major (a weight matrix [out_features, in_features])
  C  : [M, N] row-major
Blaze's own host reference takes B as [K, N] row-major (tests/test_gemm_naive.cu:38-48); the
result is the same sum in the same order, see ``gemm_f32_bkn`` and ``ref_gemm_cpu_fp16``.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_f32p = ctypes.POINTER(ctypes.c_float)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libblaze_oracle.so")
        if not os.path.exists(path):
            from . import build_oracle  # noqa: PLC0415
            build_oracle.build_oracle()
        L = ctypes.CDLL(path)
        L.blzo_quantize_fp8.restype = ctypes.c_float
        L.blzo_quantize_nvfp4.restype = ctypes.c_float
        L.blzo_amax.restype = ctypes.c_float
        _LIB = L
    return _LIB


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ------------------------------------------------------------------ formats

def f16_to_f32(x):
    x = _c(x, np.uint16); out = np.empty(x.shape, np.float32)
    _lib().blzo_f16_to_f32_n(_p(x, _u16p), _p(out, _f32p), ctypes.c_long(x.size)); return out


def f32_to_f16(x, satfinite: bool = False):
    x = _c(x, np.float32); out = np.empty(x.shape, np.uint16)
    _lib().blzo_f32_to_f16_n(_p(x, _f32p), _p(out, _u16p), ctypes.c_long(x.size), int(satfinite)); return out


def bf16_to_f32(x):
    x = _c(x, np.uint16); out = np.empty(x.shape, np.float32)
    _lib().blzo_bf16_to_f32_n(_p(x, _u16p), _p(out, _f32p), ctypes.c_long(x.size)); return out


def f32_to_bf16(x):
    x = _c(x, np.float32); out = np.empty(x.shape, np.uint16)
    _lib().blzo_f32_to_bf16_n(_p(x, _f32p), _p(out, _u16p), ctypes.c_long(x.size)); return out


def e4m3_to_f32(x):
    x = _c(x, np.uint8); out = np.empty(x.shape, np.float32)
    _lib().blzo_e4m3_to_f32_n(_p(x, _u8p), _p(out, _f32p), ctypes.c_long(x.size)); return out


def f32_to_e4m3(x):
    x = _c(x, np.float32); out = np.empty(x.shape, np.uint8)
    _lib().blzo_f32_to_e4m3_n(_p(x, _f32p), _p(out, _u8p), ctypes.c_long(x.size)); return out


def e2m1_to_f32(x):
    x = _c(x, np.uint8); out = np.empty(x.shape, np.float32)
    _lib().blzo_e2m1_to_f32_n(_p(x, _u8p), _p(out, _f32p), ctypes.c_long(x.size)); return out


def f32_to_e2m1(x):
    x = _c(x, np.float32); out = np.empty(x.shape, np.uint8)
    _lib().blzo_f32_to_e2m1_n(_p(x, _f32p), _p(out, _u8p), ctypes.c_long(x.size)); return out


def narrow(c32: np.ndarray, out_dtype: str) -> np.ndarray:
    """fp32 -> the output type's raw bits: 'f16' (saturating, as the CUDA epilogue), 'bf16', 'f32'."""
    if out_dtype == "f16":
        return f32_to_f16(c32, satfinite=True)
    if out_dtype == "bf16":
        return f32_to_bf16(c32)
    return _c(c32, np.float32)


def widen(raw: np.ndarray, out_dtype: str) -> np.ndarray:
    if out_dtype == "f16":
        return f16_to_f32(raw)
    if out_dtype == "bf16":
        return bf16_to_f32(raw)
    return _c(raw, np.float32)


# -------------------------------------------------------------- seeded fill

def fill_uniform_rand(n: int, seed: int) -> np.ndarray:
    """Blaze's test fill: srand(seed); (rand()/RAND_MAX - 0.5)*2 (tests/test_gemm_naive.cu:50-56)."""
    out = np.empty(n, np.float32)
    _lib().blzo_fill_uniform_rand(_p(out, _f32p), ctypes.c_long(n), ctypes.c_uint(seed)); return out


# -------------------------------------------------------------- quantisers

def quantize_fp8(x):
    """Per-tensor E4M3: returns (codes uint8, s) with s = 448/amax and codes = e4m3_rn(x*s)."""
    x = _c(x, np.float32); q = np.empty(x.shape, np.uint8)
    s = _lib().blzo_quantize_fp8(_p(x, _f32p), _p(q, _u8p), ctypes.c_long(x.size))
    return q, float(np.float32(s))


def quantize_nvfp4(x, g: float = 0.0):
    """Two-level NVFP4 of a [rows, K] matrix (K % 16 == 0): (data [rows,K/2], sf [rows,K/16], g)."""
    x = _c(x, np.float32); rows, K = x.shape
    assert K % 16 == 0
    data = np.empty((rows, K // 2), np.uint8); sf = np.empty((rows, K // 16), np.uint8)
    g = _lib().blzo_quantize_nvfp4(_p(x, _f32p), ctypes.c_long(rows), ctypes.c_long(K),
                                   _p(data, _u8p), _p(sf, _u8p), ctypes.c_float(g))
    return data, sf, float(np.float32(g))


def dequant_nvfp4_noglobal(data, sf) -> np.ndarray:
    """e2m1(q)*e4m3(sf) per element, [rows, K] fp32 (exact); the global scale is applied later."""
    data = _c(data, np.uint8); sf = _c(sf, np.uint8)
    rows, kh = data.shape; K = kh * 2
    out = np.empty((rows, K), np.float32)
    _lib().blzo_dequant_nvfp4_noglobal(_p(data, _u8p), _p(sf, _u8p), ctypes.c_long(rows), ctypes.c_long(K), _p(out, _f32p))
    return out


def tile_sf(sf, row_blocks: int | None = None, katoms: int | None = None) -> np.ndarray:
    """Row-major [rows, K/16] scales -> the 128x4 tiled layout the tensor-core path stages."""
    sf = _c(sf, np.uint8); rows, kb = sf.shape
    rb = row_blocks if row_blocks is not None else (rows + 127) // 128
    ka = katoms if katoms is not None else (kb + 3) // 4
    out = np.empty(rb * ka * 512, np.uint8)
    _lib().blzo_tile_sf(_p(sf, _u8p), ctypes.c_long(rows), ctypes.c_long(kb), _p(out, _u8p), ctypes.c_long(rb), ctypes.c_long(ka))
    return out


# -------------------------------------------------------------------- GEMM

def gemm_f32(A, Bt, nthreads: int = 0) -> np.ndarray:
    """C[i,j] = sum_k A[i,k]*Bt[j,k]: fp32 accumulate, k ascending, no FMA contraction."""
    A = _c(A, np.float32); Bt = _c(Bt, np.float32)
    M, K = A.shape; N, K2 = Bt.shape
    assert K == K2
    C = np.empty((M, N), np.float32)
    if nthreads <= 0:
        nthreads = os.cpu_count() or 1
    _lib().blzo_gemm_f32(_p(A, _f32p), _p(Bt, _f32p), _p(C, _f32p), ctypes.c_long(M), ctypes.c_long(N), ctypes.c_long(K), int(nthreads))
    return C


def gemm_f32_bkn(A, B) -> np.ndarray:
    """Same loop with B as [K, N] row-major, the layout Blaze's gemm_cpu_fp16 takes."""
    A = _c(A, np.float32); B = _c(B, np.float32)
    M, K = A.shape; K2, N = B.shape
    assert K == K2
    C = np.empty((M, N), np.float32)
    _lib().blzo_gemm_f32_bkn(_p(A, _f32p), _p(B, _f32p), _p(C, _f32p), ctypes.c_long(M), ctypes.c_long(N), ctypes.c_long(K))
    return C


EPILOGUES = {"none": 0, "bias": 1, "silu": 2, "bias_silu": 3, "residual": 4}


def epilogue(C32, alpha: float = 1.0, bias=None, residual=None, mode: str = "none") -> np.ndarray:
    C = np.array(C32, dtype=np.float32, order="C", copy=True)
    M, N = C.shape
    b = _c(bias, np.float32) if bias is not None else None
    r = _c(residual, np.float32) if residual is not None else None
    _lib().blzo_epilogue(_p(C, _f32p), ctypes.c_long(M), ctypes.c_long(N), ctypes.c_float(alpha),
                         _p(b, _f32p) if b is not None else None, _p(r, _f32p) if r is not None else None,
                         EPILOGUES[mode])
    return C


def swiglu(acc_gate, alpha_gate: float, acc_up, alpha_up: float) -> np.ndarray:
    """Fused gate / up projection: silu(alpha_gate * gate) * (alpha_up * up) in fp32 -- what Blaze's
    launch_fused_gate_up declares (include/gemm/mixed_gemm_sm100.cuh:87-109; SiLU as in
    src/kernels/gemm_mixed_sm100.cu:202-229)."""
    g = epilogue(acc_gate, alpha_gate, mode="silu")
    u = epilogue(acc_up, alpha_up)
    return (g * u).astype(np.float32)


def gemm_dense16(A_raw, Bt_raw, in_dtype: str, nthreads: int = 0) -> np.ndarray:
    """fp16 / bf16 operands (raw 16-bit codes) -> fp32 accumulator."""
    w = f16_to_f32 if in_dtype == "f16" else bf16_to_f32
    return gemm_f32(w(A_raw), w(Bt_raw), nthreads)


def gemm_fp8(qa, qbt, sa: float, sb: float, nthreads: int = 0):
    """E4M3 codes, per-tensor scales: returns (acc fp32, alpha) with alpha = 1/(sa*sb)."""
    acc = gemm_f32(e4m3_to_f32(qa), e4m3_to_f32(qbt), nthreads)
    alpha = float(np.float32(1.0) / (np.float32(sa) * np.float32(sb)))
    return acc, alpha


def gemm_nvfp4(a_data, a_sf, ga: float, b_data, b_sf, gb: float, nthreads: int = 0):
    """Block-scaled product: acc = sum_k (a*sfa)(b*sfb); alpha = ga*gb is applied by the epilogue."""
    acc = gemm_f32(dequant_nvfp4_noglobal(a_data, a_sf), dequant_nvfp4_noglobal(b_data, b_sf), nthreads)
    return acc, float(np.float32(ga) * np.float32(gb))


def gemm_w4a16(A_raw, in_dtype: str, b_data, b_sf, gb: float, nthreads: int = 0):
    """16-bit activations times NVFP4 weights: acc = sum_k a*(q*sf); alpha = gb."""
    w = f16_to_f32 if in_dtype == "f16" else bf16_to_f32
    acc = gemm_f32(w(A_raw), dequant_nvfp4_noglobal(b_data, b_sf), nthreads)
    return acc, float(np.float32(gb))


# ------------------------------------------ the reference's own host functions

def _ref():
    """Blaze's tests/test_gemm_naive.cu compiled as a shared object (oracle/_ref), or None."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libblaze_ref_naive.so")
        if not os.path.exists(path):
            return None
        _REF = ctypes.CDLL(path, mode=os.RTLD_LAZY)
    return _REF


def ref_available() -> bool:
    return _ref() is not None


def ref_gemm_cpu_fp16(A_f16_raw, B_f16_raw_kn) -> np.ndarray:
    """Blaze's gemm_cpu_fp16(A [M,K] fp16, B [K,N] fp16) -> C [M,N] fp32, single thread."""
    L = _ref()
    A = _c(A_f16_raw, np.uint16); B = _c(B_f16_raw_kn, np.uint16)
    M, K = A.shape; K2, N = B.shape
    assert K == K2
    C = np.empty((M, N), np.float32)
    fn = getattr(L, "_Z13gemm_cpu_fp16PK6__halfS1_Pfiii")
    fn(A.ctypes.data_as(ctypes.c_void_p), B.ctypes.data_as(ctypes.c_void_p), _p(C, _f32p), int(M), int(N), int(K))
    return C


def ref_init_random_fp16(n: int, seed: int) -> np.ndarray:
    """Blaze's init_random_fp16(data, size, seed) -> raw fp16 codes."""
    L = _ref()
    out = np.empty(n, np.uint16)
    fn = getattr(L, "_Z16init_random_fp16P6__halfij")
    fn(out.ctypes.data_as(ctypes.c_void_p), int(n), ctypes.c_uint(seed))
    return out
