// launch_fused_gate_up through namespace blaze (include/gemm/blaze_gemm.cuh), with weights in
// Blaze's Fp4WeightTensor convention: data [K, N/2] (even column in the low nibble), block scales
// [K/16, N], one fp32 scale per tensor.  Blaze declares the function
// (include/gemm/mixed_gemm_sm100.cuh:87-109) and leaves its body a stub, so the expected values come
// from first principles: every operand is chosen so that all products and sums are exact in fp32.
//   x[m][k]      = 0.125 * (m % 4 + 1)
//   gate[k][n]   = E2M1 code 1 + n % 3   (0.5, 1.0, 1.5), scale 1.0 (0x38), tensor scale 0.5
//   up[k][n]     = E2M1 code 2 + n % 2   (1.0, 1.5), scale 2.0 (0x40) where (n / 16) is odd else 1.0, tensor scale 0.25
//   out[m][n]    = silu(K * x * gate * 0.5) * (K * x * up * sf * 0.25)
// Prints "PASS" / "FAIL ..." and returns 0 / 1.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <vector>

#include "gemm/blaze_gemm.cuh"

static bool run_case(int M, int N, int K) {
    static const float e2m1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    std::vector<half> x(static_cast<size_t>(M) * K);
    for (int m = 0; m < M; ++m) for (int k = 0; k < K; ++k) x[static_cast<size_t>(m) * K + k] = __float2half(0.125f * (m % 4 + 1));
    std::vector<uint8_t> gd(static_cast<size_t>(K) * N / 2), ud(gd.size()), gs(static_cast<size_t>(K / 16) * N), us(gs.size());
    auto gcode = [](int n) { return 1 + n % 3; };
    auto ucode = [](int n) { return 2 + n % 2; };
    auto usf = [](int n) { return (n / 16) % 2 ? 2.0f : 1.0f; };
    for (int k = 0; k < K; ++k)
        for (int n = 0; n < N; n += 2) {
            gd[static_cast<size_t>(k) * (N / 2) + n / 2] = static_cast<uint8_t>(gcode(n) | (gcode(n + 1) << 4));
            ud[static_cast<size_t>(k) * (N / 2) + n / 2] = static_cast<uint8_t>(ucode(n) | (ucode(n + 1) << 4));
        }
    for (int kb = 0; kb < K / 16; ++kb)
        for (int n = 0; n < N; ++n) {
            gs[static_cast<size_t>(kb) * N + n] = 0x38;
            us[static_cast<size_t>(kb) * N + n] = usf(n) == 2.0f ? 0x40 : 0x38;
        }
    half *dx = nullptr, *dout = nullptr;
    uint8_t *dgd = nullptr, *dud = nullptr, *dgs = nullptr, *dus = nullptr;
    if (cudaMalloc(&dx, x.size() * 2) || cudaMalloc(&dout, static_cast<size_t>(M) * N * 2) || cudaMalloc(&dgd, gd.size()) || cudaMalloc(&dud, ud.size()) ||
        cudaMalloc(&dgs, gs.size()) || cudaMalloc(&dus, us.size())) { std::printf("FAIL cudaMalloc\n"); return false; }
    cudaMemcpy(dx, x.data(), x.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dgd, gd.data(), gd.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(dud, ud.data(), ud.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(dgs, gs.data(), gs.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(dus, us.data(), us.size(), cudaMemcpyHostToDevice);
    cudaMemset(dout, 0xFF, static_cast<size_t>(M) * N * 2);
    blaze::Fp4WeightTensor Wg{dgd, reinterpret_cast<const __nv_fp8_e4m3*>(dgs), 0.5f, K, N};
    blaze::Fp4WeightTensor Wu{dud, reinterpret_cast<const __nv_fp8_e4m3*>(dus), 0.25f, K, N};
    blaze::launch_fused_gate_up(dx, Wg, Wu, dout, M, N, K, 0);
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { std::printf("FAIL %s\n", cudaGetErrorString(e)); return false; }
    std::vector<half> out(static_cast<size_t>(M) * N);
    cudaMemcpy(out.data(), dout, out.size() * 2, cudaMemcpyDeviceToHost);
    int bad = 0;
    for (int m = 0; m < M && bad < 5; ++m)
        for (int n = 0; n < N && bad < 5; ++n) {
            const double xv = 0.125 * (m % 4 + 1);
            const double g = K * xv * e2m1[gcode(n)] * 0.5, u = K * xv * e2m1[ucode(n)] * usf(n) * 0.25;
            const double want = g / (1.0 + std::exp(-g)) * u;
            const double got = __half2float(out[static_cast<size_t>(m) * N + n]);
            if (!(std::fabs(got - want) <= 2e-3 * std::fmax(std::fabs(want), 1.0))) {      // fp16 rounding of the result: 2^-11 relative
                std::printf("FAIL M=%d N=%d K=%d out[%d][%d] = %g, expected %g\n", M, N, K, m, n, got, want);
                ++bad;
            }
        }
    cudaFree(dx); cudaFree(dout); cudaFree(dgd); cudaFree(dud); cudaFree(dgs); cudaFree(dus);
    return bad == 0;
}

int main() {
    // one kernel (N a multiple of 16): a few rows, a ragged tile, several tiles; then the two-GEMM form (N = 40)
    if (!run_case(3, 48, 64) || !run_case(200, 208, 128) || !run_case(520, 1024, 256) || !run_case(5, 40, 64)) return 1;
    std::printf("PASS\n");
    return 0;
}
