"""ctypes binding of libblaze_b200.so (the C ABI of include/blaze_b200.h).

There is no fallback: if the shared library is missing or a symbol is absent, importing callers
get an exception that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# BLAZE_B200_LIBRARY points at another build of the same library (e.g. a tuning build).
LIB_PATH = os.environ.get("BLAZE_B200_LIBRARY") or os.path.join(_HERE, "libblaze_b200.so")

# enums of blaze_b200.h
OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_NO_DEVICE, ERR_TOO_LARGE, ERR_OUT_OF_MEMORY = range(8)
GEMM_F16, GEMM_BF16, GEMM_FP8, GEMM_NVFP4, GEMM_W4A16_F16, GEMM_W4A16_BF16 = range(6)
F16, BF16, F32 = range(3)
EPI_NONE, EPI_BIAS, EPI_SILU, EPI_BIAS_SILU, EPI_RESIDUAL_ADD, EPI_SWIGLU = range(6)
B_KMAJOR, B_NMAJOR = range(2)
SF_ROWMAJOR, SF_TILED = range(2)
FLAG_CLC_SCHEDULER, FLAG_STATIC_WEIGHTS, FLAG_TAIL_SPLIT = 1, 2, 4
VARIANT_AUTO, VARIANT_TILE_128x128, VARIANT_PAIR_256x256, VARIANT_DECODE, VARIANT_QUAD_512x256, VARIANT_PAIR_256x384, VARIANT_PAIR_256x128 = range(7)

KINDS = {"f16": GEMM_F16, "bf16": GEMM_BF16, "fp8": GEMM_FP8, "nvfp4": GEMM_NVFP4,
         "w4a16_f16": GEMM_W4A16_F16, "w4a16_bf16": GEMM_W4A16_BF16}
DTYPES = {"f16": F16, "bf16": BF16, "f32": F32}
EPILOGUES = {"none": EPI_NONE, "bias": EPI_BIAS, "silu": EPI_SILU, "bias_silu": EPI_BIAS_SILU, "residual": EPI_RESIDUAL_ADD, "swiglu": EPI_SWIGLU}
VARIANTS = {"auto": VARIANT_AUTO, "128x128": VARIANT_TILE_128x128, "256x256": VARIANT_PAIR_256x256, "decode": VARIANT_DECODE, "512x256": VARIANT_QUAD_512x256, "256x384": VARIANT_PAIR_256x384,
            "256x128": VARIANT_PAIR_256x128}

# every symbol include/blaze_b200.h declares
EXPORTS = (
    "blz_version", "blz_status_string", "blz_last_cuda_error", "blz_last_cuda_error_string",
    "blz_gemm_plan_create", "blz_gemm_execute", "blz_gemm_plan_set_a", "blz_gemm_plan_check",
    "blz_gemm_plan_info", "blz_gemm_plan_refresh_weights", "blz_gemm_plan_destroy", "blz_gemm_launch",
    "blz_amax", "blz_quantize_fp8", "blz_quantize_nvfp4", "blz_tiled_scales_bytes", "blz_tile_scales", "blz_interleave_gate_up",
    "blz_gemm_nvfp4_decode_static",
    "blz_peer_buffer_create", "blz_peer_buffer_open", "blz_peer_buffer_close", "blz_peer_buffer_destroy", "blz_gemm_execute_gather",
    "blz_wait_probe",
    "blz_shard_bounds", "blz_nccl_unique_id", "blz_sharded_plan_create", "blz_sharded_plan_info", "blz_sharded_plan_output_handle",
    "blz_sharded_plan_connect", "blz_sharded_plan_execute", "blz_sharded_plan_check", "blz_sharded_plan_destroy", "blz_sharded_last_error",
)
EXCHANGE_NONE, EXCHANGE_NCCL, EXCHANGE_PEER_STORES = range(3)
EXCHANGES = {"none": EXCHANGE_NONE, "nccl": EXCHANGE_NCCL, "peer_stores": EXCHANGE_PEER_STORES}


class GemmDesc(ctypes.Structure):
    _fields_ = [
        ("kind", ctypes.c_int32), ("out_dtype", ctypes.c_int32), ("epilogue", ctypes.c_int32), ("variant", ctypes.c_int32),
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
        ("b_layout", ctypes.c_int32), ("a_sf_layout", ctypes.c_int32), ("b_sf_layout", ctypes.c_int32),
        ("A", ctypes.c_void_p), ("A_sf", ctypes.c_void_p), ("B", ctypes.c_void_p), ("B_sf", ctypes.c_void_p),
        ("a_scale", ctypes.c_float), ("b_scale", ctypes.c_float),
        ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("ldc", ctypes.c_int64),
        ("b_scale2", ctypes.c_float), ("flags", ctypes.c_int32),
    ]


class PlanInfo(ctypes.Structure):
    _fields_ = [
        ("variant", ctypes.c_int32), ("tile_m", ctypes.c_int32), ("tile_n", ctypes.c_int32), ("stages", ctypes.c_int32),
        ("split_k", ctypes.c_int32), ("grid", ctypes.c_int32), ("smem_bytes", ctypes.c_int32), ("tmem_cols", ctypes.c_int32),
        ("launches", ctypes.c_int32), ("scheduler", ctypes.c_int32), ("workspace_bytes", ctypes.c_int64),
        ("tail_tiles", ctypes.c_int32), ("tail_split", ctypes.c_int32),
    ]


class ShardedDesc(ctypes.Structure):
    _fields_ = [("gemm", GemmDesc), ("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("exchange", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("nccl_id", ctypes.c_char_p)]


class ShardedInfo(ctypes.Structure):
    _fields_ = [("col_lo", ctypes.c_int64), ("col_hi", ctypes.c_int64), ("exchange", ctypes.c_int32), ("world", ctypes.c_int32),
                ("rank", ctypes.c_int32), ("reserved", ctypes.c_int32), ("own_output", ctypes.c_void_p), ("gemm", PlanInfo)]


class BlazeError(RuntimeError):
    def __init__(self, where: str, status: int, detail: str = ""):
        self.status = status
        super().__init__("%s: status %d (%s)%s" % (where, status, status_string(status), (" -- " + detail) if detail else ""))


_LIB = None


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "blaze_b200: %s is missing. Build it with `python -m blaze_b200.build` (needs nvcc); "
            "there is no CPU or PyTorch fallback." % LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(L, name):
            raise RuntimeError("blaze_b200: %s does not export %s; rebuild it" % (LIB_PATH, name))
    vp, i32, i64, f32p = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.POINTER(ctypes.c_float)
    L.blz_version.restype = ctypes.c_int
    L.blz_status_string.restype = ctypes.c_char_p
    L.blz_status_string.argtypes = [ctypes.c_int]
    L.blz_last_cuda_error.restype = ctypes.c_int
    L.blz_last_cuda_error_string.restype = ctypes.c_char_p
    L.blz_gemm_plan_create.argtypes = [ctypes.POINTER(GemmDesc), ctypes.POINTER(vp)]
    L.blz_gemm_execute.argtypes = [vp, vp, vp]
    L.blz_gemm_plan_set_a.argtypes = [vp, vp, vp, ctypes.c_float]
    L.blz_gemm_plan_check.argtypes = [vp, vp]
    L.blz_gemm_plan_info.argtypes = [vp, ctypes.POINTER(PlanInfo)]
    L.blz_gemm_plan_refresh_weights.argtypes = [vp, vp]
    L.blz_gemm_plan_refresh_weights.restype = ctypes.c_int
    L.blz_gemm_plan_destroy.argtypes = [vp]
    L.blz_gemm_launch.argtypes = [ctypes.POINTER(GemmDesc), vp, vp]
    L.blz_amax.argtypes = [vp, i32, i64, vp, vp]
    L.blz_quantize_fp8.argtypes = [vp, i32, i64, vp, vp, vp, vp]
    L.blz_quantize_nvfp4.argtypes = [vp, i32, i64, i64, vp, vp, vp, i32, vp, vp]
    L.blz_tiled_scales_bytes.restype = i64
    L.blz_tiled_scales_bytes.argtypes = [i64, i64]
    L.blz_tile_scales.argtypes = [vp, i64, i64, i64, i64, vp, vp]
    L.blz_interleave_gate_up.argtypes = [vp, vp, vp, i64, i64, vp]
    L.blz_interleave_gate_up.restype = ctypes.c_int
    L.blz_gemm_nvfp4_decode_static.argtypes = [vp, vp, ctypes.c_float, vp, vp, ctypes.c_float, i32, i32, i32, vp, i32, i64, vp, vp]
    L.blz_gemm_nvfp4_decode_static.restype = ctypes.c_int
    L.blz_peer_buffer_create.argtypes = [i64, ctypes.POINTER(vp), ctypes.c_char_p]
    L.blz_peer_buffer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.blz_peer_buffer_close.argtypes = [vp]
    L.blz_peer_buffer_destroy.argtypes = [vp]
    L.blz_gemm_execute_gather.argtypes = [vp, i32, ctypes.POINTER(vp), i64, i64, vp]
    L.blz_wait_probe.argtypes = [ctypes.c_uint64, vp, vp, vp]
    L.blz_wait_probe.restype = ctypes.c_int
    for name in ("blz_peer_buffer_create", "blz_peer_buffer_open", "blz_peer_buffer_close", "blz_peer_buffer_destroy", "blz_gemm_execute_gather"):
        getattr(L, name).restype = ctypes.c_int
    for name in ("blz_gemm_plan_create", "blz_gemm_execute", "blz_gemm_plan_set_a", "blz_gemm_plan_check", "blz_gemm_plan_info",
                 "blz_gemm_plan_destroy", "blz_gemm_launch", "blz_amax", "blz_quantize_fp8", "blz_quantize_nvfp4", "blz_tile_scales"):
        getattr(L, name).restype = ctypes.c_int
    L.blz_shard_bounds.argtypes = [i64, i32, i32, i32, ctypes.POINTER(i64), ctypes.POINTER(i64)]
    L.blz_nccl_unique_id.argtypes = [ctypes.c_char_p]
    L.blz_sharded_plan_create.argtypes = [ctypes.POINTER(ShardedDesc), ctypes.POINTER(vp)]
    L.blz_sharded_plan_info.argtypes = [vp, ctypes.POINTER(ShardedInfo)]
    L.blz_sharded_plan_output_handle.argtypes = [vp, ctypes.c_char_p]
    L.blz_sharded_plan_connect.argtypes = [vp, ctypes.c_char_p]
    L.blz_sharded_plan_execute.argtypes = [vp, vp, vp]
    L.blz_sharded_plan_check.argtypes = [vp, vp]
    L.blz_sharded_plan_destroy.argtypes = [vp]
    L.blz_sharded_last_error.restype = ctypes.c_char_p
    for name in ("blz_shard_bounds", "blz_nccl_unique_id", "blz_sharded_plan_create", "blz_sharded_plan_info", "blz_sharded_plan_output_handle",
                 "blz_sharded_plan_connect", "blz_sharded_plan_execute", "blz_sharded_plan_check", "blz_sharded_plan_destroy"):
        getattr(L, name).restype = ctypes.c_int
    _ = f32p
    _LIB = L
    return L


def status_string(status: int) -> str:
    return lib().blz_status_string(int(status)).decode()


def check(where: str, status: int) -> None:
    if status != OK:
        raise BlazeError(where, status, lib().blz_last_cuda_error_string().decode())
