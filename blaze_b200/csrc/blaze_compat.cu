// blaze_compat.cu -- namespace blaze entry points (include/gemm/blaze_gemm.cuh) as shims over the
// C ABI.  Argument meaning and ownership follow Blaze's host code: launch_* sets everything up,
// runs once and releases it (src/kernels/gemm_fp8_sm100.cu:268-334); create_* builds a reusable
// plan, execute_* only launches, destroy_*(nullptr) is a no-op (gemm_fp8_sm100.cu:340-430).
// Errors go to stderr and the call returns, as Blaze's launchers do (gemm_fp8_sm100.cu:308-312).
#include <cstdio>

#include "../../include/blaze_b200.h"
#include "../../include/gemm/blaze_gemm.cuh"

namespace {

void report(const char* where, blz_status s) {
    if (s != BLZ_OK) fprintf(stderr, "blaze: %s failed: %s (%s)\n", where, blz_status_string(s), blz_last_cuda_error_string());
}

blz_gemm_desc base_desc(int kind, int M, int N, int K, int epilogue, const void* bias, const void* residual) {
    blz_gemm_desc d = {};
    d.kind = kind;
    d.out_dtype = BLZ_F16;
    d.epilogue = epilogue;
    d.variant = BLZ_VARIANT_AUTO;
    d.M = M; d.N = N; d.K = K;
    d.b_layout = BLZ_B_NMAJOR;       // Blaze passes B as [K, N] row-major
    d.a_sf_layout = BLZ_SF_ROWMAJOR;
    d.b_sf_layout = BLZ_SF_ROWMAJOR;
    d.a_scale = 1.0f; d.b_scale = 1.0f;
    d.bias = bias; d.residual = residual;
    d.ldc = 0;
    return d;
}

template <typename TA, typename TB>
blz_gemm_desc fp4_desc(const TA& A, const TB& B, int M, int N, int K, int epilogue, const void* bias) {
    blz_gemm_desc d = base_desc(BLZ_GEMM_NVFP4, M, N, K, epilogue, bias, nullptr);
    d.A = A.data; d.A_sf = A.block_scales; d.a_scale = A.tensor_scale;
    d.B = B.data; d.B_sf = B.block_scales; d.b_scale = B.tensor_scale;
    return d;
}

blz_gemm_desc mixed_desc(const half* A, const blaze::Fp4WeightTensor& B, int M, int N, int K, int epilogue, const void* bias, const void* residual) {
    blz_gemm_desc d = base_desc(BLZ_GEMM_W4A16_F16, M, N, K, epilogue, bias, residual);
    d.A = A;
    d.B = B.data; d.B_sf = B.block_scales; d.b_scale = B.tensor_scale;
    return d;
}

template <typename PlanT>
PlanT* make_plan(const blz_gemm_desc& d, const char* where) {
    blz_gemm_plan* p = nullptr;
    blz_status s = blz_gemm_plan_create(&d, &p);
    report(where, s);
    return reinterpret_cast<PlanT*>(p);
}

void run_plan(void* plan, void* C, cudaStream_t stream, const char* where) {
    if (!plan) { fprintf(stderr, "blaze: %s called with a null plan\n", where); return; }
    report(where, blz_gemm_execute(reinterpret_cast<blz_gemm_plan*>(plan), C, stream));
}

void run_once(const blz_gemm_desc& d, void* C, cudaStream_t stream, const char* where) {
    report(where, blz_gemm_launch(&d, C, stream));
}

__global__ void multiply_inplace_kernel(half* __restrict__ out, const half* __restrict__ gate, long long n) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = __float2half_rn(__half2float(out[i]) * __half2float(gate[i]));
}

}  // namespace

namespace blaze {

// ---------------------------------------------------------------- FP8
void launch_gemm_fp8(const __nv_fp8_e4m3* A, const __nv_fp8_e4m3* B, half* C, int M, int N, int K, const half* bias, GemmEpilogue epilogue, cudaStream_t stream) {
    blz_gemm_desc d = base_desc(BLZ_GEMM_FP8, M, N, K, static_cast<int>(epilogue), bias, nullptr);
    d.A = A; d.B = B;
    run_once(d, C, stream, "launch_gemm_fp8");
}
Fp8GemmPlan* create_fp8_gemm_plan(const __nv_fp8_e4m3* A, const __nv_fp8_e4m3* B, int M, int N, int K, const half* bias, GemmEpilogue epilogue) {
    blz_gemm_desc d = base_desc(BLZ_GEMM_FP8, M, N, K, static_cast<int>(epilogue), bias, nullptr);
    d.A = A; d.B = B;
    return make_plan<Fp8GemmPlan>(d, "create_fp8_gemm_plan");
}
void execute_fp8_gemm(Fp8GemmPlan* plan, half* C, cudaStream_t stream) { run_plan(plan, C, stream, "execute_fp8_gemm"); }
void destroy_fp8_gemm_plan(Fp8GemmPlan* plan) { blz_gemm_plan_destroy(reinterpret_cast<blz_gemm_plan*>(plan)); }

// ---------------------------------------------------------------- NVFP4
void launch_gemm_fp4(const Fp4WeightTensor& A, const Fp4WeightTensor& B, half* C, int M, int N, int K, const half* bias, Fp4Epilogue epilogue, cudaStream_t stream) {
    run_once(fp4_desc(A, B, M, N, K, static_cast<int>(epilogue), bias), C, stream, "launch_gemm_fp4");
}
Fp4GemmPlan* create_fp4_gemm_plan(const Fp4WeightTensor& A, const Fp4WeightTensor& B, int M, int N, int K, const half* bias, Fp4Epilogue epilogue) {
    return make_plan<Fp4GemmPlan>(fp4_desc(A, B, M, N, K, static_cast<int>(epilogue), bias), "create_fp4_gemm_plan");
}
void execute_fp4_gemm(Fp4GemmPlan* plan, half* C, cudaStream_t stream) { run_plan(plan, C, stream, "execute_fp4_gemm"); }
void destroy_fp4_gemm_plan(Fp4GemmPlan* plan) { blz_gemm_plan_destroy(reinterpret_cast<blz_gemm_plan*>(plan)); }

void launch_gemm_fp4_blkscaled(const Fp4BlkScaledWeightTensor& A, const Fp4BlkScaledWeightTensor& B, half* C, int M, int N, int K, const half* bias, Fp4BlkScaledEpilogue epilogue, cudaStream_t stream) {
    run_once(fp4_desc(A, B, M, N, K, static_cast<int>(epilogue), bias), C, stream, "launch_gemm_fp4_blkscaled");
}
Fp4BlkScaledGemmPlan* create_fp4_blkscaled_gemm_plan(const Fp4BlkScaledWeightTensor& A, const Fp4BlkScaledWeightTensor& B, int M, int N, int K, const half* bias, Fp4BlkScaledEpilogue epilogue) {
    return make_plan<Fp4BlkScaledGemmPlan>(fp4_desc(A, B, M, N, K, static_cast<int>(epilogue), bias), "create_fp4_blkscaled_gemm_plan");
}
void execute_fp4_blkscaled_gemm(Fp4BlkScaledGemmPlan* plan, half* C, cudaStream_t stream) { run_plan(plan, C, stream, "execute_fp4_blkscaled_gemm"); }
void destroy_fp4_blkscaled_gemm_plan(Fp4BlkScaledGemmPlan* plan) { blz_gemm_plan_destroy(reinterpret_cast<blz_gemm_plan*>(plan)); }

// Every kernel behind this library is persistent, so the two block-scaled families share one path.
void launch_gemm_fp4_blkscaled_persistent(const Fp4BlkScaledWeightTensor& A, const Fp4BlkScaledWeightTensor& B, half* C, int M, int N, int K, const half* bias, Fp4BlkScaledEpilogue epilogue, cudaStream_t stream) {
    run_once(fp4_desc(A, B, M, N, K, static_cast<int>(epilogue), bias), C, stream, "launch_gemm_fp4_blkscaled_persistent");
}
Fp4BlkScaledPersistentGemmPlan* create_fp4_blkscaled_persistent_gemm_plan(const Fp4BlkScaledWeightTensor& A, const Fp4BlkScaledWeightTensor& B, int M, int N, int K, const half* bias, Fp4BlkScaledEpilogue epilogue) {
    return make_plan<Fp4BlkScaledPersistentGemmPlan>(fp4_desc(A, B, M, N, K, static_cast<int>(epilogue), bias), "create_fp4_blkscaled_persistent_gemm_plan");
}
void execute_fp4_blkscaled_persistent_gemm(Fp4BlkScaledPersistentGemmPlan* plan, half* C, cudaStream_t stream) { run_plan(plan, C, stream, "execute_fp4_blkscaled_persistent_gemm"); }
void destroy_fp4_blkscaled_persistent_gemm_plan(Fp4BlkScaledPersistentGemmPlan* plan) { blz_gemm_plan_destroy(reinterpret_cast<blz_gemm_plan*>(plan)); }

// ---------------------------------------------------------------- W4A16
void launch_gemm_mixed(const half* A, const Fp4WeightTensor& B, half* C, int M, int N, int K, const half* bias, const half* residual, MixedEpilogue epilogue, cudaStream_t stream) {
    run_once(mixed_desc(A, B, M, N, K, static_cast<int>(epilogue), bias, residual), C, stream, "launch_gemm_mixed");
}
MixedGemmPlan* create_mixed_gemm_plan(const half* A, const Fp4WeightTensor& B, int M, int N, int K, const half* bias, const half* residual, MixedEpilogue epilogue) {
    // Blaze's plan converts its operands once, at creation (src/kernels/gemm_mixed_sm100.cu:412-470): the weights handed
    // to a plan are static for the plan's life, so the 16-bit copy of larger problems is made here and not per execute
    blz_gemm_desc d = mixed_desc(A, B, M, N, K, static_cast<int>(epilogue), bias, residual);
    d.flags |= BLZ_FLAG_STATIC_WEIGHTS;
    return make_plan<MixedGemmPlan>(d, "create_mixed_gemm_plan");
}
void execute_mixed_gemm(MixedGemmPlan* plan, half* C, cudaStream_t stream) { run_plan(plan, C, stream, "execute_mixed_gemm"); }
void destroy_mixed_gemm_plan(MixedGemmPlan* plan) { blz_gemm_plan_destroy(reinterpret_cast<blz_gemm_plan*>(plan)); }

// output = SiLU(x W_gate) * (x W_up).  One GEMM over the 2N interleaved gate / up columns whose
// epilogue multiplies the pairs (BLZ_EPI_SWIGLU); the interleaved copy of the packed weights and
// their scales is made here per call, as launch_* owns no state.  N not a multiple of 16: two
// GEMMs (the gate one applies SiLU) and one elementwise pass.
void launch_fused_gate_up(const half* x, const Fp4WeightTensor& W_gate, const Fp4WeightTensor& W_up, half* output, int M, int N, int K, cudaStream_t stream) {
    if (N % 16 == 0 && K % 32 == 0) {
        const long long data_bytes = static_cast<long long>(K) * (N / 2), sf_bytes = static_cast<long long>(K / 16) * N;
        uint8_t *data = nullptr, *sf = nullptr;
        if (cudaMalloc(&data, static_cast<size_t>(2 * data_bytes)) != cudaSuccess || cudaMalloc(&sf, static_cast<size_t>(2 * sf_bytes)) != cudaSuccess) {
            (void)cudaGetLastError();
            cudaFree(data);
            fprintf(stderr, "blaze: launch_fused_gate_up could not allocate %lld bytes\n", 2 * (data_bytes + sf_bytes));
            return;
        }
        // [K, N/2] bytes: 16 columns = 8 bytes per group; [K/16, N] scales: 16 bytes per group
        report("launch_fused_gate_up(interleave)", blz_interleave_gate_up(W_gate.data, W_up.data, data, data_bytes / 8, 8, stream));
        report("launch_fused_gate_up(interleave)", blz_interleave_gate_up(W_gate.block_scales, W_up.block_scales, sf, sf_bytes / 16, 16, stream));
        blz_gemm_desc d = base_desc(BLZ_GEMM_W4A16_F16, M, 2 * N, K, BLZ_EPI_SWIGLU, nullptr, nullptr);
        d.A = x; d.B = data; d.B_sf = sf;
        d.b_scale = W_gate.tensor_scale; d.b_scale2 = W_up.tensor_scale;
        run_once(d, output, stream, "launch_fused_gate_up");      // synchronises the stream
        cudaFree(data); cudaFree(sf);
        return;
    }
    half* gate = nullptr;
    const long long n = static_cast<long long>(M) * N;
    if (cudaMalloc(&gate, static_cast<size_t>(n) * sizeof(half)) != cudaSuccess) {
        (void)cudaGetLastError();
        fprintf(stderr, "blaze: launch_fused_gate_up could not allocate %lld bytes\n", n * 2);
        return;
    }
    run_once(mixed_desc(x, W_gate, M, N, K, BLZ_EPI_SILU, nullptr, nullptr), gate, stream, "launch_fused_gate_up(gate)");
    run_once(mixed_desc(x, W_up, M, N, K, BLZ_EPI_NONE, nullptr, nullptr), output, stream, "launch_fused_gate_up(up)");
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    multiply_inplace_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(output, gate, n);
    cudaStreamSynchronize(stream);
    cudaFree(gate);
}

// ---------------------------------------------------------------- dense fp16
void launch_gemm_fp16(const half* A, const half* B_colmajor, float* C, int M, int N, int K, cudaStream_t stream) {
    blz_gemm_desc d = base_desc(BLZ_GEMM_F16, M, N, K, BLZ_EPI_NONE, nullptr, nullptr);
    d.out_dtype = BLZ_F32; d.b_layout = BLZ_B_KMAJOR; d.A = A; d.B = B_colmajor;
    run_once(d, C, stream, "launch_gemm_fp16");
}
Fp16GemmPlan* create_fp16_gemm_plan(const half* A, const half* B_colmajor, int M, int N, int K) {
    blz_gemm_desc d = base_desc(BLZ_GEMM_F16, M, N, K, BLZ_EPI_NONE, nullptr, nullptr);
    d.out_dtype = BLZ_F32; d.b_layout = BLZ_B_KMAJOR; d.A = A; d.B = B_colmajor;
    return make_plan<Fp16GemmPlan>(d, "create_fp16_gemm_plan");
}
void execute_fp16_gemm(Fp16GemmPlan* plan, float* C, cudaStream_t stream) { run_plan(plan, C, stream, "execute_fp16_gemm"); }
void destroy_fp16_gemm_plan(Fp16GemmPlan* plan) { blz_gemm_plan_destroy(reinterpret_cast<blz_gemm_plan*>(plan)); }

}  // namespace blaze
