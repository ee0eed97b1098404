// common.cuh -- what the GEMM kernels share: operand / epilogue enums, the epilogue parameter block
// and its arithmetic (alpha -> bias -> SiLU / residual -> narrow, the order of Blaze's
// src/kernels/gemm_mixed_sm100.cu:202-229).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

// Per-role cycle counters and an event trace exist in tuning builds only (-DBLZ_KERNEL_TIMING pulls in
// tuning_counters.cuh); in the library as shipped the hooks below expand to nothing.
#ifdef BLZ_KERNEL_TIMING
#include "tuning_counters.cuh"
#else
#define BLZ_T_DECL(name)
#define BLZ_T_NOW() 0
#define BLZ_T_ADD(acc, t0)
#define BLZ_T_STORE(slot, v)
#define BLZ_T_STORE_IF(cond, slot, v)
#define BLZ_TRACE(region, i)
#endif

namespace blz {

enum MmaKind : int { MMA_F16 = 0, MMA_F8 = 1, MMA_NVF4 = 2, MMA_W4A16 = 3 };   // W4A16: kind::f16 instructions, B expanded from NVFP4 in the kernel
enum OutType : int { OUT_F16 = 0, OUT_BF16 = 1, OUT_F32 = 2 };
enum EpiMode : int { EPI_NONE = 0, EPI_BIAS = 1, EPI_SILU = 2, EPI_BIAS_SILU = 3, EPI_RESIDUAL = 4, EPI_SWIGLU = 5 };
// EPI_SWIGLU: the GEMM's N columns are gate / up projections interleaved in groups of 16 (columns
// 32b .. 32b+15 gate, 32b+16 .. 32b+31 up, of outputs 16b .. 16b+15); C is [M, N/2]:
// C[m, 16b+i] = silu(alpha * acc[32b+i]) * (alpha2 * acc[32b+16+i]).  What Blaze declares as
// launch_fused_gate_up (include/gemm/mixed_gemm_sm100.cuh:87-109; its body is a stub,
// src/kernels/gemm_mixed_sm100.cu:520-543).

struct EpilogueParams {
    void* C;                 // [M, ldc] in the output type
    const void* bias;        // [N] in the output type (fp32 when the output is fp32), or null
    const void* residual;    // [M, ldr] in the output type, or null
    long long ldc, ldr;      // row pitches in elements
    float alpha;
    float alpha2;            // EPI_SWIGLU: multiplier of the up columns
    int mode;                // EpiMode
    int out_type;            // OutType
    int vec_ok;              // rows of C (and residual) are 16-byte aligned: wide stores allowed
};


__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + __expf(-v)); }

// fp32 -> fp16 with finite overflow clamped to +-65504 (NaN stays NaN)
__device__ __forceinline__ float clamp_f16_range(float v) {
    return (v != v) ? v : fminf(fmaxf(v, -65504.0f), 65504.0f);
}

template <int OUT> struct OutElem;
template <> struct OutElem<OUT_F16> { using type = __half; };
template <> struct OutElem<OUT_BF16> { using type = __nv_bfloat16; };
template <> struct OutElem<OUT_F32> { using type = float; };

template <int OUT> __device__ __forceinline__ float load_out_elem(const void* p, long long i) {
    if constexpr (OUT == OUT_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
    else if constexpr (OUT == OUT_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    else return reinterpret_cast<const float*>(p)[i];
}

// Applies the epilogue to 32 consecutive accumulator columns of one row and stores them.
//   acc: raw fp32 bits from tensor memory; row / col0: position in C.
// EPI_SWIGLU on one 32-column group of the GEMM (col0 a multiple of 32): 16 outputs at column col0 / 2.
template <int OUT>
__device__ __forceinline__ void epilogue_store_swiglu32(const EpilogueParams& e, const uint32_t (&acc)[32], int row, int col0, int N) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = silu_f32(__uint_as_float(acc[i]) * e.alpha) * (__uint_as_float(acc[16 + i]) * e.alpha2);
    using T = typename OutElem<OUT>::type;
    const int ocol = col0 >> 1, n_out = N >> 1;
    T* dst = reinterpret_cast<T*>(e.C) + static_cast<long long>(row) * e.ldc + ocol;
    if (ocol + 16 <= n_out && e.vec_ok) {
        if constexpr (OUT == OUT_F32) {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if constexpr (OUT == OUT_F16) {
                        __half2 h = __floats2half2_rn(clamp_f16_range(v[i + 2 * j]), clamp_f16_range(v[i + 2 * j + 1]));
                        w[j] = *reinterpret_cast<uint32_t*>(&h);
                    } else {
                        __nv_bfloat162 h = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                        w[j] = *reinterpret_cast<uint32_t*>(&h);
                    }
                }
                *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (ocol + i < n_out) {
                if constexpr (OUT == OUT_F16) dst[i] = __float2half_rn(clamp_f16_range(v[i]));
                else if constexpr (OUT == OUT_BF16) dst[i] = __float2bfloat16_rn(v[i]);
                else dst[i] = v[i];
            }
        }
    }
}

template <int OUT>
__device__ __forceinline__ void epilogue_store32(const EpilogueParams& e, const uint32_t (&acc)[32], int row, int col0, int M, int N) {
    if (row >= M || col0 >= N) return;
    if (e.mode == EPI_SWIGLU) { epilogue_store_swiglu32<OUT>(e, acc, row, col0, N); return; }
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]) * e.alpha;
    const bool full = (col0 + 32 <= N);
    if (e.mode == EPI_BIAS || e.mode == EPI_BIAS_SILU) {
        if (e.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (full || col0 + i < N) v[i] += load_out_elem<OUT>(e.bias, col0 + i);
        }
    }
    if (e.mode == EPI_SILU || e.mode == EPI_BIAS_SILU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = silu_f32(v[i]);
    }
    if (e.mode == EPI_RESIDUAL && e.residual != nullptr) {
        const long long roff = static_cast<long long>(row) * e.ldr + col0;
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (full || col0 + i < N) v[i] += load_out_elem<OUT>(e.residual, roff + i);
    }
    using T = typename OutElem<OUT>::type;
    T* dst = reinterpret_cast<T*>(e.C) + static_cast<long long>(row) * e.ldc + col0;
    if (full && e.vec_ok) {
        if constexpr (OUT == OUT_F32) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if constexpr (OUT == OUT_F16) {
                        __half2 h = __floats2half2_rn(clamp_f16_range(v[i + 2 * j]), clamp_f16_range(v[i + 2 * j + 1]));
                        w[j] = *reinterpret_cast<uint32_t*>(&h);
                    } else {
                        __nv_bfloat162 h = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                        w[j] = *reinterpret_cast<uint32_t*>(&h);
                    }
                }
                *reinterpret_cast<uint4*>(dst + i) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (col0 + i < N) {
                if constexpr (OUT == OUT_F16) dst[i] = __float2half_rn(clamp_f16_range(v[i]));
                else if constexpr (OUT == OUT_BF16) dst[i] = __float2bfloat16_rn(v[i]);
                else dst[i] = v[i];
            }
        }
    }
}

// alpha, bias, SiLU, residual on 32 consecutive accumulator columns of one row (fp32 in, fp32 out);
// bias / residual are read in the output's element type and only inside the matrix.
__device__ __forceinline__ void epilogue_math32(const EpilogueParams& e, const uint32_t (&acc)[32], float (&v)[32], int row, int col0, int M, int N) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]) * e.alpha;
    if (e.mode == EPI_NONE) return;
    const bool has_bias = (e.mode == EPI_BIAS || e.mode == EPI_BIAS_SILU) && e.bias != nullptr;
    const bool has_res = e.mode == EPI_RESIDUAL && e.residual != nullptr && row < M;
    const long long roff = static_cast<long long>(row) * e.ldr + col0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if (col0 + i < N) {
            if (has_bias) v[i] += e.out_type == OUT_BF16 ? load_out_elem<OUT_BF16>(e.bias, col0 + i) : e.out_type == OUT_F16 ? load_out_elem<OUT_F16>(e.bias, col0 + i) : load_out_elem<OUT_F32>(e.bias, col0 + i);
            if (has_res) v[i] += e.out_type == OUT_BF16 ? load_out_elem<OUT_BF16>(e.residual, roff + i) : e.out_type == OUT_F16 ? load_out_elem<OUT_F16>(e.residual, roff + i) : load_out_elem<OUT_F32>(e.residual, roff + i);
        }
    }
    if (e.mode == EPI_SILU || e.mode == EPI_BIAS_SILU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = silu_f32(v[i]);
    }
}

// two fp32 values -> one 32-bit word of two fp16 (saturating) or bf16 values
__device__ __forceinline__ uint32_t pack2_out(int out_type, float a, float b) {
    if (out_type == OUT_F16) {
        __half2 h = __floats2half2_rn(clamp_f16_range(a), clamp_f16_range(b));
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void epilogue_store32_dyn(const EpilogueParams& e, const uint32_t (&acc)[32], int row, int col0, int M, int N) {
    if (e.out_type == OUT_BF16) epilogue_store32<OUT_BF16>(e, acc, row, col0, M, N);
    else if (e.out_type == OUT_F16) epilogue_store32<OUT_F16>(e, acc, row, col0, M, N);
    else epilogue_store32<OUT_F32>(e, acc, row, col0, M, N);
}

// W4A16, tiled kernel: 256 threads turn one stage of packed weights (128 rows x 64 K values) into
// the 16-bit operand tile.  Thread t takes half a row (32 values = 16 packed bytes, two block
// scales).  packed: [128][32] bytes, even k in the low nibble; sf_atom: the tiled scale layout,
// row r at byte (r % 32) * 16 + (r / 32) * 4; dst: shared-memory address of the operand tile
// (1024-byte aligned), 16-byte unit j of row r at unit j ^ (r % 8), as a 128-byte-swizzled TMA
// load would have left it.  q * scale has at most six significant bits: exact in fp16 and bf16.
// bf16: the fp16 bit pattern of an E2M1 value, shifted right by three with the sign put back,
// read as bf16 is the value times 2^-112; the scale is prepared as bf16(scale * 2^112).
template <bool BF16>
__device__ __forceinline__ void expand_w4_stage(const uint8_t* packed, const uint8_t* sf_atom, uint32_t dst, int t) {
    const int row = t >> 1, half = t & 1;
    const uint4 w = *reinterpret_cast<const uint4*>(packed + row * 32 + half * 16);
    const uint32_t sf4 = *reinterpret_cast<const uint32_t*>(sf_atom + (row & 31) * 16 + (row >> 5) * 4);
    const uint32_t s01 = cvt_e4m3x2_to_f16x2(static_cast<uint16_t>(sf4 >> (16 * half)));
    uint32_t s_lo, s_hi;
    if constexpr (BF16) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&s01));
        const float big = __uint_as_float(0x77800000u);                    // 2^112
        s_lo = pack_bf16x2(f.x * big, f.x * big);
        s_hi = pack_bf16x2(f.y * big, f.y * big);
    } else {
        s_lo = __byte_perm(s01, 0, 0x1010); s_hi = __byte_perm(s01, 0, 0x3232);
    }
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    const uint32_t drow = dst + row * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t s = c < 2 ? s_lo : s_hi;
        uint32_t h[4], o[4];
        cvt_e2m1x8_to_f16x2x4(words[c], h);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if constexpr (BF16) o[b] = mul_bf16x2(((h[b] >> 3) & 0x0FFF0FFFu) | (h[b] & 0x80008000u), s);
            else o[b] = mul_f16x2(h[b], s);
        }
        const uint32_t addr = drow + (static_cast<uint32_t>((half * 4 + c) ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
    }
}

__host__ __device__ constexpr uint32_t tmem_cols_pow2(uint32_t need) {
    return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
}

}  // namespace blz
