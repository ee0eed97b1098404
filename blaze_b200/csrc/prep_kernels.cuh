// prep_kernels.cuh -- operand preparation around the GEMM: scale-factor tiling, layout
// repacking for operands given in Blaze's [K, N] convention, quantisers and the NVFP4 -> 16-bit
// dequantiser.  All HBM-bound byte work: one pass, coalesced, grid sized by the problem.
//
// Counterparts in Blaze: interleave_scales_kernel / interleave_scales_transposed_kernel
// (src/kernels/gemm_fp4_blkscaled_sm100.cu:59-104) and fp16_to_e4m3_kernel
// (src/kernels/gemm_mixed_sm100.cu:312-321).  Blaze has no quantiser; the arithmetic here is
// the definition the CPU oracle states, operation for operation, so results are bit-identical.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace blz {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ uint8_t f32_to_e4m3_bits(float v) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_bits_to_f32(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
    return __half2float(__half(h));
}
__device__ __forceinline__ uint8_t f32_to_e2m1_bits(float v) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp4(v, __NV_E2M1, cudaRoundNearest)) & 0xF;
}
// magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 with the sign in bit 3
__device__ __forceinline__ float e2m1_bits_to_f32(uint32_t n) {
    const uint32_t e = (n >> 1) & 3u, m = n & 1u;
    float v = (e == 0) ? 0.5f * static_cast<float>(m) : __uint_as_float(((e + 126u) << 23) | (m << 22));
    return (n & 8u) ? -v : v;
}

// byte offset of the scale of (row r, 16-value K block b) in the tiled layout
__host__ __device__ __forceinline__ long long tiled_sf_offset(long long r, long long b, long long katoms) {
    return ((r / 128) * katoms + b / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4);
}

// ---- scale tiling: in(r, b) = sf[r*row_stride + b*blk_stride]; `tiled` was zeroed beforehand.
__global__ void tile_scales_kernel(const uint8_t* __restrict__ sf, long long rows, long long kblocks,
                                   long long row_stride, long long blk_stride, long long katoms,
                                   uint8_t* __restrict__ tiled) {
    const long long total = rows * kblocks;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        long long r, b;
        if (blk_stride == 1) { r = i / kblocks; b = i % kblocks; }   // consecutive threads walk the contiguous dimension
        else { b = i / rows; r = i % rows; }
        tiled[tiled_sf_offset(r, b, katoms)] = sf[r * row_stride + b * blk_stride];
    }
}

// ---- [K, N] -> [N, K] for 1- or 2-byte elements (shared-memory tile transpose)
template <typename T>
__global__ void transpose_kn_to_nk_kernel(const T* __restrict__ in, T* __restrict__ out, int K, int N) {
    __shared__ T tile[32][33];
    const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int k = k0 + j, n = n0 + threadIdx.x;
        if (k < K && n < N) tile[j][threadIdx.x] = in[static_cast<long long>(k) * N + n];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int n = n0 + j, k = k0 + threadIdx.x;
        if (n < N && k < K) out[static_cast<long long>(n) * K + k] = tile[threadIdx.x][j];
    }
}

// ---- packed E2M1 [K, N/2] (two N-neighbours per byte, even N in the low nibble)
//      -> [N, K/2] (two K-neighbours per byte, even K in the low nibble)
__global__ void repack_fp4_kn_to_nk_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int K, int N) {
    // one thread per output byte pair: handles n = 2*np, 2*np+1 and k = 2*kp, 2*kp+1
    const long long total = static_cast<long long>(N / 2) * (K / 2);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int np = static_cast<int>(i % (N / 2)), kp = static_cast<int>(i / (N / 2));
        const uint8_t r0 = in[static_cast<long long>(2 * kp) * (N / 2) + np];       // k even: n even (lo), n odd (hi)
        const uint8_t r1 = in[static_cast<long long>(2 * kp + 1) * (N / 2) + np];   // k odd
        out[static_cast<long long>(2 * np) * (K / 2) + kp] = static_cast<uint8_t>((r0 & 0xF) | ((r1 & 0xF) << 4));
        out[static_cast<long long>(2 * np + 1) * (K / 2) + kp] = static_cast<uint8_t>((r0 >> 4) | (r1 & 0xF0));
    }
}

// ---- amax: |x| maximum, combined into *out with an integer max on the bit pattern
template <typename T>
__global__ void amax_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
    float m = 0.0f;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        m = fmaxf(m, fabsf(to_f32<T>(x[i])));
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float wm[32];
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < (blockDim.x >> 5) ? wm[threadIdx.x] : 0.0f;
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(m));
    }
}

// ---- FP8 per tensor: s = 448/amax (1 when amax == 0); q = e4m3_rn(x*s); scales = {s, 1/s}
template <typename T>
__global__ void quantize_fp8_kernel(const T* __restrict__ x, long long n, const float* __restrict__ amax,
                                    uint8_t* __restrict__ q, float* __restrict__ scales) {
    const float am = *amax;
    const float s = am > 0.0f ? __fdiv_rn(448.0f, am) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0 && scales != nullptr) { scales[0] = s; scales[1] = __fdiv_rn(1.0f, s); }
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        q[i] = f32_to_e4m3_bits(__fmul_rn(to_f32<T>(x[i]), s));
}

// ---- NVFP4: one thread per 16-value block
template <typename T>
__global__ void quantize_nvfp4_kernel(const T* __restrict__ x, long long rows, long long K, const float* __restrict__ amax,
                                      uint8_t* __restrict__ data, uint8_t* __restrict__ sf, int tiled, long long katoms,
                                      float* __restrict__ g_out) {
    const float am_all = *amax;
    const float g = am_all > 0.0f ? __fdiv_rn(am_all, 2688.0f) : 1.0f;   // 6 * 448
    if (blockIdx.x == 0 && threadIdx.x == 0 && g_out != nullptr) *g_out = g;
    const long long kb = K / 16, total = rows * kb;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / kb, b = i % kb;
        const T* p = x + r * K + b * 16;
        float v[16];
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) { v[j] = to_f32<T>(p[j]); am = fmaxf(am, fabsf(v[j])); }
        const uint8_t s8 = f32_to_e4m3_bits(__fdiv_rn(__fdiv_rn(am, 6.0f), g));
        const float sfv = e4m3_bits_to_f32(s8);
        sf[tiled ? tiled_sf_offset(r, b, katoms) : (r * kb + b)] = s8;
        const float d = __fmul_rn(g, sfv);
        uint32_t w[2] = {0u, 0u};
        if (sfv != 0.0f) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                w[j >> 3] |= static_cast<uint32_t>(f32_to_e2m1_bits(__fdiv_rn(v[j], d))) << (4 * (j & 7));
        }
        *reinterpret_cast<uint2*>(data + r * (K / 2) + b * 8) = make_uint2(w[0], w[1]);
    }
}

// ---- NVFP4 weights -> 16-bit values q*sf (exact: 6 significant bits), global scale left out.
//      data [rows, K/2], sf read through the tiled layout; out [rows, K].
//      One thread per 8 values: 4 packed bytes in, 16 bytes out, so a warp reads 128 and writes 512
//      contiguous bytes per instruction; hardware conversions (fp16: cvt + packed multiply; bf16:
//      the fp16 pattern shifted by three is the value x 2^-112, multiplied by bf16(scale x 2^112)).
template <bool BF16>
__global__ void dequant_nvfp4_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ sf_tiled, long long katoms,
                                     long long rows, long long K, uint16_t* __restrict__ out) {
    const long long k8 = K / 8, total = rows * k8;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / k8, c = i % k8;                      // c: which group of 8 values of the row
        const uint32_t s8 = sf_tiled[tiled_sf_offset(r, c >> 1, katoms)];
        const uint32_t w = *reinterpret_cast<const uint32_t*>(data + r * (K / 2) + c * 4);
        const uint32_t s1 = cvt_e4m3x2_to_f16x2(static_cast<uint16_t>(s8));          // low half = the scale
        uint32_t s;
        if constexpr (BF16) {
            const float f = __half2float(__ushort_as_half(static_cast<unsigned short>(s1 & 0xFFFFu))) * __uint_as_float(0x77800000u);   // x 2^112
            s = pack_bf16x2(f, f);
        } else {
            s = __byte_perm(s1, 0, 0x1010);
        }
        uint32_t h[4], o[4];
        cvt_e2m1x8_to_f16x2x4(w, h);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if constexpr (BF16) o[j] = mul_bf16x2(((h[j] >> 3) & 0x0FFF0FFFu) | (h[j] & 0x80008000u), s);
            else o[j] = mul_f16x2(h[j], s);
        }
        *reinterpret_cast<uint4*>(out + r * K + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---- split-K, tiled kernel: C = epilogue(alpha * sum_s partial[s]) ; partial: [splits][rows_per_split][pitch] fp32,
//      summed in split order (fixed, so results do not depend on timing).  One thread per 4 columns.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, long long rows_per_split, long long pitch,
                                     int M, int N, EpilogueParams e) {
    const long long groups = (static_cast<long long>(N) + 3) / 4, total = static_cast<long long>(M) * groups;
    const int esize = e.out_type == OUT_F32 ? 4 : 2;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long m = i / groups;
        const int n0 = static_cast<int>(i % groups) * 4;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int sidx = 0; sidx < splits; ++sidx) {
            const float4 t = *reinterpret_cast<const float4*>(partial + (sidx * rows_per_split + m) * pitch + n0);
            v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int n = n0 + t;
            v[t] *= e.alpha;
            if (n < N && e.mode != EPI_NONE) {
                if ((e.mode == EPI_BIAS || e.mode == EPI_BIAS_SILU) && e.bias != nullptr)
                    v[t] += e.out_type == OUT_BF16 ? load_out_elem<OUT_BF16>(e.bias, n) : e.out_type == OUT_F16 ? load_out_elem<OUT_F16>(e.bias, n) : load_out_elem<OUT_F32>(e.bias, n);
                if (e.mode == EPI_SILU || e.mode == EPI_BIAS_SILU) v[t] = silu_f32(v[t]);
                if (e.mode == EPI_RESIDUAL && e.residual != nullptr) {
                    const long long roff = m * e.ldr + n;
                    v[t] += e.out_type == OUT_BF16 ? load_out_elem<OUT_BF16>(e.residual, roff) : e.out_type == OUT_F16 ? load_out_elem<OUT_F16>(e.residual, roff) : load_out_elem<OUT_F32>(e.residual, roff);
                }
            }
        }
        uint8_t* dst = reinterpret_cast<uint8_t*>(e.C) + (m * e.ldc + n0) * esize;
        const bool whole = n0 + 4 <= N && (reinterpret_cast<uintptr_t>(dst) & (esize == 4 ? 15u : 7u)) == 0;
        if (e.out_type == OUT_F32) {
            if (whole) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            else for (int t = 0; t < 4 && n0 + t < N; ++t) reinterpret_cast<float*>(dst)[t] = v[t];
        } else {
            const uint32_t w0 = pack2_out(e.out_type, v[0], v[1]), w1 = pack2_out(e.out_type, v[2], v[3]);
            if (whole) *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
            else for (int t = 0; t < 4 && n0 + t < N; ++t) reinterpret_cast<uint16_t*>(dst)[t] = static_cast<uint16_t>((t < 2 ? w0 : w1) >> (16 * (t & 1)));
        }
    }
}

// out = 4-byte words of groups taken alternately from `a` and `b`: group g of a, group g of b, ...
// (words_per_group words each).  Builds the gate / up interleaved weights of the EPI_SWIGLU epilogue.
__global__ void interleave_groups_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, uint32_t* __restrict__ out,
                                         long long n_groups, long long words_per_group) {
    const long long total = n_groups * words_per_group;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long g = i / words_per_group, w = i - g * words_per_group;
        out[(2 * g) * words_per_group + w] = a[i];
        out[(2 * g + 1) * words_per_group + w] = b[i];
    }
}

}  // namespace blz
