// blaze_gemm.cuh -- the C++ host API of namespace blaze, as Blaze's own programs call it
// (tests/test_gemm.cu:138,206,287,371,471; benchmarks/bench_gemm.cu:209-440), implemented as thin
// shims over the C ABI of blaze_b200.h.  Names, argument order, default arguments and ownership
// follow Blaze's headers:
//   include/gemm/fp8_gemm_sm100.cuh:43-99, fp4_gemm_sm100.cuh:26-129,
//   fp4_blkscaled_gemm_sm100.cuh:43-208, mixed_gemm_sm100.cuh:56-139.
// Data pointers are device pointers owned by the caller and must outlive a plan; C is given at
// execute time; destroy(nullptr) is a no-op.  Output is fp16 as in Blaze (other output types are
// reached through the C ABI).  Differences, all toward Blaze's stated intent:
//   - B arrives in Blaze's [K, N] row-major convention and is repacked K-major when the plan is
//     built (4-bit B: two N-neighbours per byte; block scales [K/16, N]);
//   - block scales are applied by every FP4 path (Blaze's f8f6f4 kernels stage and ignore them);
//   - the mixed GEMM keeps fp16 activations instead of casting them to E4M3;
//   - the fp16 store saturates to +-65504 instead of producing infinities;
//   - failures are reported on stderr and the call returns; nothing calls exit().
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace blaze {

constexpr float FP4_E2M1_MAX = 6.0f;
constexpr int FP4_BLOCK_SIZE = 16;            // values per E4M3 block scale
constexpr int FP4_BLKSCALED_BLOCK_SIZE = 16;

// Tile shapes of the kernels behind each entry point (informational).
struct Fp8GemmConfig { static constexpr int TILE_M = 256, TILE_N = 256, TILE_K = 128, BLOCK_SIZE = 256, PIPELINE_STAGES = 6; };
struct Fp4GemmConfig { static constexpr int TILE_M = 256, TILE_N = 256, TILE_K = 256, BLOCK_SIZE = 384, PIPELINE_STAGES = 5; };
struct Fp4BlkScaledConfig {
    static constexpr int TILE_M = 256, TILE_N = 256, TILE_K = 256, K_PER_MMA = 64, BLOCK_SIZE = 384, PIPELINE_STAGES = 5;
    static constexpr int SF_VEC_SIZE = 16;
};
struct MixedGemmConfig { static constexpr int TILE_M = 256, TILE_N = 256, TILE_K = 64, BLOCK_SIZE = 256, PIPELINE_STAGES = 6; };

enum class GemmEpilogue { NONE, BIAS, SILU, BIAS_SILU };
enum class Fp4Epilogue { NONE, BIAS, SILU, BIAS_SILU };
enum class Fp4BlkScaledEpilogue { NONE, BIAS, SILU, BIAS_SILU };
enum class MixedEpilogue { NONE, BIAS, SILU, BIAS_SILU, RESIDUAL_ADD };

// NVFP4 operand: packed E2M1 (two per byte), one E4M3 scale per 16 values along K, one fp32
// scale per tensor.  As operand A: data [M, K/2], scales [M, K/16].  As operand B: data
// [K, N/2], scales [K/16, N].
struct Fp4WeightTensor {
    const uint8_t* data;
    const __nv_fp8_e4m3* block_scales;
    float tensor_scale;
    int rows;
    int cols;
};
struct Fp4BlkScaledWeightTensor {
    const uint8_t* data;
    const __nv_fp8_e4m3* block_scales;
    float tensor_scale;
    int rows;
    int cols;
};

struct Fp8GemmPlan;
struct Fp4GemmPlan;
struct Fp4BlkScaledGemmPlan;
struct Fp4BlkScaledPersistentGemmPlan;
struct MixedGemmPlan;
struct Fp16GemmPlan;

// ---- E4M3 x E4M3 -> fp16 (A [M,K], B [K,N], row-major)
void launch_gemm_fp8(const __nv_fp8_e4m3* A, const __nv_fp8_e4m3* B, half* C, int M, int N, int K,
                     const half* bias = nullptr, GemmEpilogue epilogue = GemmEpilogue::NONE, cudaStream_t stream = 0);
Fp8GemmPlan* create_fp8_gemm_plan(const __nv_fp8_e4m3* A, const __nv_fp8_e4m3* B, int M, int N, int K,
                                  const half* bias = nullptr, GemmEpilogue epilogue = GemmEpilogue::NONE);
void execute_fp8_gemm(Fp8GemmPlan* plan, half* C, cudaStream_t stream = 0);
void destroy_fp8_gemm_plan(Fp8GemmPlan* plan);

// ---- NVFP4 x NVFP4 -> fp16
void launch_gemm_fp4(const Fp4WeightTensor& A, const Fp4WeightTensor& B, half* C, int M, int N, int K,
                     const half* bias = nullptr, Fp4Epilogue epilogue = Fp4Epilogue::NONE, cudaStream_t stream = 0);
Fp4GemmPlan* create_fp4_gemm_plan(const Fp4WeightTensor& A, const Fp4WeightTensor& B, int M, int N, int K,
                                  const half* bias = nullptr, Fp4Epilogue epilogue = Fp4Epilogue::NONE);
void execute_fp4_gemm(Fp4GemmPlan* plan, half* C, cudaStream_t stream = 0);
void destroy_fp4_gemm_plan(Fp4GemmPlan* plan);

void launch_gemm_fp4_blkscaled(const Fp4BlkScaledWeightTensor& A, const Fp4BlkScaledWeightTensor& B, half* C, int M, int N, int K,
                               const half* bias = nullptr, Fp4BlkScaledEpilogue epilogue = Fp4BlkScaledEpilogue::NONE,
                               cudaStream_t stream = 0);
Fp4BlkScaledGemmPlan* create_fp4_blkscaled_gemm_plan(const Fp4BlkScaledWeightTensor& A, const Fp4BlkScaledWeightTensor& B, int M, int N, int K,
                                                     const half* bias = nullptr,
                                                     Fp4BlkScaledEpilogue epilogue = Fp4BlkScaledEpilogue::NONE);
void execute_fp4_blkscaled_gemm(Fp4BlkScaledGemmPlan* plan, half* C, cudaStream_t stream = 0);
void destroy_fp4_blkscaled_gemm_plan(Fp4BlkScaledGemmPlan* plan);

void launch_gemm_fp4_blkscaled_persistent(const Fp4BlkScaledWeightTensor& A, const Fp4BlkScaledWeightTensor& B, half* C, int M, int N, int K,
                                          const half* bias = nullptr, Fp4BlkScaledEpilogue epilogue = Fp4BlkScaledEpilogue::NONE,
                                          cudaStream_t stream = 0);
Fp4BlkScaledPersistentGemmPlan* create_fp4_blkscaled_persistent_gemm_plan(const Fp4BlkScaledWeightTensor& A, const Fp4BlkScaledWeightTensor& B,
                                                                          int M, int N, int K, const half* bias = nullptr,
                                                                          Fp4BlkScaledEpilogue epilogue = Fp4BlkScaledEpilogue::NONE);
void execute_fp4_blkscaled_persistent_gemm(Fp4BlkScaledPersistentGemmPlan* plan, half* C, cudaStream_t stream = 0);
void destroy_fp4_blkscaled_persistent_gemm_plan(Fp4BlkScaledPersistentGemmPlan* plan);

// ---- fp16 activations x NVFP4 weights -> fp16
void launch_gemm_mixed(const half* A, const Fp4WeightTensor& B, half* C, int M, int N, int K, const half* bias = nullptr,
                       const half* residual = nullptr, MixedEpilogue epilogue = MixedEpilogue::NONE, cudaStream_t stream = 0);
// output = SiLU(x W_gate) * (x W_up)
void launch_fused_gate_up(const half* x, const Fp4WeightTensor& W_gate, const Fp4WeightTensor& W_up, half* output, int M, int N, int K,
                          cudaStream_t stream = 0);
MixedGemmPlan* create_mixed_gemm_plan(const half* A, const Fp4WeightTensor& B, int M, int N, int K, const half* bias = nullptr,
                                      const half* residual = nullptr, MixedEpilogue epilogue = MixedEpilogue::NONE);
void execute_mixed_gemm(MixedGemmPlan* plan, half* C, cudaStream_t stream = 0);
void destroy_mixed_gemm_plan(MixedGemmPlan* plan);

// ---- dense fp16 x fp16 -> fp32 on the tensor cores (no counterpart among Blaze's entry points:
//      its fp16 GEMM is a CUDA-core bring-up program, src/kernels/gemm_fp16_naive.cu).
//      A [M,K] row-major, B column-major (stored [N,K]), C [M,N] fp32.
void launch_gemm_fp16(const half* A, const half* B_colmajor, float* C, int M, int N, int K, cudaStream_t stream = 0);
Fp16GemmPlan* create_fp16_gemm_plan(const half* A, const half* B_colmajor, int M, int N, int K);
void execute_fp16_gemm(Fp16GemmPlan* plan, float* C, cudaStream_t stream = 0);
void destroy_fp16_gemm_plan(Fp16GemmPlan* plan);

}  // namespace blaze
