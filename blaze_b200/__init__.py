"""blaze_b200 -- B200 (sm_100a) GEMM hot path of Blaze behind Blaze's own host API.

The product is the CUDA library (blaze_b200/libblaze_b200.so, C ABI in include/blaze_b200.h);
this package is the Python host-side mirror used by the tests and the bench.
"""
from . import _native
from .gemm import (GemmPlan, amax, gemm_nvfp4_decode_static, create_fp4_blkscaled_gemm_plan, create_fp4_blkscaled_persistent_gemm_plan,
                   create_fp4_gemm_plan, create_fp8_gemm_plan, create_fp16_gemm_plan, create_mixed_gemm_plan,
                   create_fused_gate_up_plan, interleave_gate_up,
                   destroy_fp4_blkscaled_gemm_plan, destroy_fp4_blkscaled_persistent_gemm_plan, destroy_fp4_gemm_plan,
                   destroy_fp8_gemm_plan, destroy_fp16_gemm_plan, destroy_mixed_gemm_plan, execute_fp4_blkscaled_gemm,
                   execute_fp4_blkscaled_persistent_gemm, execute_fp4_gemm, execute_fp8_gemm, execute_fp16_gemm,
                   execute_mixed_gemm, quantize_fp8, quantize_nvfp4, tile_scales, tiled_scales_bytes)
from ._native import BlazeError

__all__ = [n for n in dir() if not n.startswith("_")]
