// gemm_kernel.cuh -- persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M,N] = epilogue( alpha * sum_k A[M,K] * B[N,K]^T )        (both operands K-major)
//
// One CTA per SM walks output tiles of 128 x BN.  Warp roles:
//   warp 0   TMA producer: per 128-byte K stage loads the A tile, the B tile and (NVFP4) the
//            scale-factor atoms into a ring of shared-memory stages
//   warp 1   MMA issuer: one thread copies scale factors smem -> tensor memory and issues four
//            tcgen05.mma (32 bytes of K each) per stage; tcgen05.commit frees the stage and, after
//            the last stage, publishes the accumulator
//   warp 2   allocates / frees tensor memory
//   warps 4-7 epilogue: tcgen05.ld the fp32 accumulator (one row per thread), apply
//            alpha / bias / SiLU / residual, narrow, store.  With two accumulator buffers the
//            epilogue of tile i overlaps the mainloop of tile i+1.
//
// This is the counterpart of Blaze's gemm_fp8_kernel (src/kernels/gemm_fp8_sm100.cu:204-264) and
// gemm_fp4_blkscaled_persistent_kernel (src/kernels/gemm_fp4_blkscaled_sm100.cu:507-624): same
// arithmetic, different pipeline (deep TMA ring, commit-based barriers, static tile schedule,
// double-buffered accumulators, bounded waits).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace blz {

enum MmaKind : int { MMA_F16 = 0, MMA_F8 = 1, MMA_NVF4 = 2 };
enum OutType : int { OUT_F16 = 0, OUT_BF16 = 1, OUT_F32 = 2 };
enum EpiMode : int { EPI_NONE = 0, EPI_BIAS = 1, EPI_SILU = 2, EPI_BIAS_SILU = 3, EPI_RESIDUAL = 4 };

struct EpilogueParams {
    void* C;                 // [M, ldc] in the output type
    const void* bias;        // [N] in the output type (fp32 when the output is fp32), or null
    const void* residual;    // [M, ldr] in the output type, or null
    long long ldc, ldr;      // row pitches in elements
    float alpha;
    int mode;                // EpiMode
    int out_type;            // OutType
    int vec_ok;              // rows of C (and residual) are 16-byte aligned: wide stores allowed
};

struct GemmKernelParams {
    int M, N;
    int m_tiles, n_tiles;
    int k_stages;            // ceil(K bytes per row / 128)
    uint32_t idesc;
    const uint8_t* sfa;      // tiled scale factors of A: [m_tiles][sf_katoms][512]
    const uint8_t* sfb;      // tiled scale factors of B: [row blocks of 128][sf_katoms][512]
    int sf_katoms;           // 64-element K atoms per row block, padded to a multiple of 4
    EpilogueParams epi;
    int* status;             // device error word, 0 = fine
};

// Optional per-role cycle accounting, compiled in only with -DBLZ_KERNEL_TIMING (a tuning build):
// slot layout per CTA, 16 x u64: 0 producer wait-empty, 1 producer total, 2 mma wait-full,
// 3 mma wait-accumulator, 4 mma total, 5 epilogue wait-full, 6 epilogue work, 7 epilogue total, 8 tiles.
#ifdef BLZ_KERNEL_TIMING
__device__ unsigned long long g_blz_timing[1024 * 16];
#define BLZ_T_DECL(name) long long name = 0
#define BLZ_T_NOW() clock64()
#define BLZ_T_ADD(acc, t0) acc += clock64() - (t0)
#define BLZ_T_STORE(slot, v) g_blz_timing[(blockIdx.x & 1023) * 16 + (slot)] = static_cast<unsigned long long>(v)
#else
#define BLZ_T_DECL(name)
#define BLZ_T_NOW() 0
#define BLZ_T_ADD(acc, t0)
#define BLZ_T_STORE(slot, v)
#endif

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
template <int OUT>
__device__ __forceinline__ void epilogue_store32(const EpilogueParams& e, const uint32_t (&acc)[32], int row, int col0, int M, int N) {
    if (row >= M || col0 >= N) return;
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

__host__ __device__ constexpr uint32_t tmem_cols_pow2(uint32_t need) {
    return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
}

template <int KIND, int BN, int STAGES, int ACC_BUFS>
struct GemmTileConfig {
    static constexpr int BM = 128;
    static constexpr bool HAS_SF = (KIND == MMA_NVF4);
    static constexpr uint32_t A_BYTES = BM * 128;
    static constexpr uint32_t B_BYTES = BN * 128;
    static constexpr uint32_t SF_ROWBLOCK_BYTES = 4 * 512;             // four 64-element K atoms per stage
    static constexpr uint32_t SFA_BYTES = HAS_SF ? SF_ROWBLOCK_BYTES : 0;
    static constexpr uint32_t SFB_BYTES = HAS_SF ? (BN / 128) * SF_ROWBLOCK_BYTES : 0;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    static constexpr uint32_t ACC_COLS = ACC_BUFS * BN;
    static constexpr uint32_t SFA_COL = ACC_COLS;                      // 4 columns per K atom
    static constexpr uint32_t SFB_COL = ACC_COLS + 16;                 // BN/32 columns per K atom
    static constexpr uint32_t TMEM_NEED = ACC_COLS + (HAS_SF ? 16 + 4 * (BN / 32) : 0);
    static constexpr uint32_t TMEM_COLS = tmem_cols_pow2(TMEM_NEED);
    static constexpr uint32_t BAR_BYTES = 8 * (2 * STAGES + 2 * ACC_BUFS) + 16;
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
    static_assert(TMEM_NEED <= 512, "accumulators and scale factors exceed tensor memory");
    static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "invalid MMA N");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
};

template <int KIND, int BN, int STAGES, int ACC_BUFS>
__global__ void __launch_bounds__(256, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmKernelParams p) {
    using Cfg = GemmTileConfig<KIND, BN, STAGES, ACC_BUFS>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - raw);

    const uint32_t bar_base = base + STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + ACC_BUFS + b); };
    const uint32_t slot_off = STAGES * Cfg::STAGE_BYTES + 8u * (2 * STAGES + 2 * ACC_BUFS);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + slot_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + slot_off + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < ACC_BUFS; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), 4); }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 2) {
        tmem_alloc(base + slot_off, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = p.m_tiles * p.n_tiles;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            BLZ_T_DECL(t_wait); BLZ_T_DECL(t_total);
            [[maybe_unused]] const long long t_begin = BLZ_T_NOW();
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
                for (int ks = 0; ks < p.k_stages; ++ks) {
                    [[maybe_unused]] const long long t0 = BLZ_T_NOW();
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; ok = false; break;
                    }
                    BLZ_T_ADD(t_wait, t0);
                    const uint32_t sa = base + stage * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    mbar_arrive_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
                    tma_load_2d(sa, &tm_a, ks * 128, m_tile * 128, full_bar(stage));
                    tma_load_2d(sb, &tm_b, ks * 128, n_tile * BN, full_bar(stage));
                    if constexpr (Cfg::HAS_SF) {
                        const uint32_t ssfa = sb + Cfg::B_BYTES;
                        const uint32_t ssfb = ssfa + Cfg::SFA_BYTES;
                        const size_t katom = static_cast<size_t>(ks) * 4;
                        bulk_load_1d(ssfa, p.sfa + (static_cast<size_t>(m_tile) * p.sf_katoms + katom) * 512, Cfg::SF_ROWBLOCK_BYTES, full_bar(stage));
#pragma unroll
                        for (int blk = 0; blk < BN / 128; ++blk) {
                            const size_t rb = static_cast<size_t>(n_tile) * (BN / 128) + blk;
                            bulk_load_1d(ssfb + blk * Cfg::SF_ROWBLOCK_BYTES, p.sfb + (rb * p.sf_katoms + katom) * 512, Cfg::SF_ROWBLOCK_BYTES, full_bar(stage));
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            BLZ_T_ADD(t_total, t_begin);
            BLZ_T_STORE(0, t_wait); BLZ_T_STORE(1, t_total);
        }
        __syncwarp();
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            BLZ_T_DECL(t_wait_full); BLZ_T_DECL(t_wait_acc); BLZ_T_DECL(t_total);
            [[maybe_unused]] const long long t_begin = BLZ_T_NOW();
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
                const int buf = it % ACC_BUFS;
                const uint32_t use = static_cast<uint32_t>(it / ACC_BUFS);
                [[maybe_unused]] const long long ta = BLZ_T_NOW();
                if (!mbar_wait(acc_empty_bar(buf), (use & 1u) ^ 1u, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_ACC); *abort_flag = 1; ok = false; break;
                }
                BLZ_T_ADD(t_wait_acc, ta);
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int ks = 0; ks < p.k_stages; ++ks) {
                    [[maybe_unused]] const long long tf = BLZ_T_NOW();
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                    }
                    BLZ_T_ADD(t_wait_full, tf);
                    tc_fence_after_sync();
                    const uint32_t sa = base + stage * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    if constexpr (Cfg::HAS_SF) {
                        const uint32_t ssfa = sb + Cfg::B_BYTES;
                        const uint32_t ssfb = ssfa + Cfg::SFA_BYTES;
#pragma unroll
                        for (int a = 0; a < 4; ++a)
                            tc_copy_sf(tmem_base + Cfg::SFA_COL + 4 * a, make_desc_sf(ssfa + a * 512));
#pragma unroll
                        for (int blk = 0; blk < BN / 128; ++blk)
#pragma unroll
                            for (int a = 0; a < 4; ++a)
                                tc_copy_sf(tmem_base + Cfg::SFB_COL + a * (BN / 32) + blk * 4,
                                           make_desc_sf(ssfb + blk * Cfg::SF_ROWBLOCK_BYTES + a * 512));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t ad = make_desc_k_sw128(sa + k * 32);
                        const uint64_t bd = make_desc_k_sw128(sb + k * 32);
                        const uint32_t accumulate = (ks | k) != 0 ? 1u : 0u;
                        if constexpr (KIND == MMA_F16) umma_f16(d_tmem, ad, bd, p.idesc, accumulate);
                        else if constexpr (KIND == MMA_F8) umma_f8(d_tmem, ad, bd, p.idesc, accumulate);
                        else umma_nvf4(d_tmem, ad, bd, p.idesc, tmem_base + Cfg::SFA_COL + 4 * k,
                                       tmem_base + Cfg::SFB_COL + k * (BN / 32), accumulate);
                    }
                    tc_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) tc_commit(acc_full_bar(buf));
            }
            BLZ_T_ADD(t_total, t_begin);
            BLZ_T_STORE(2, t_wait_full); BLZ_T_STORE(3, t_wait_acc); BLZ_T_STORE(4, t_total); BLZ_T_STORE(8, it);
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;
        int it = 0;
        bool ok = true;
        BLZ_T_DECL(t_wait); BLZ_T_DECL(t_work); BLZ_T_DECL(t_total);
        [[maybe_unused]] const long long t_begin = BLZ_T_NOW();
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
            const int buf = it % ACC_BUFS;
            const uint32_t use = static_cast<uint32_t>(it / ACC_BUFS);
            [[maybe_unused]] const long long tw = BLZ_T_NOW();
            if (!mbar_wait(acc_full_bar(buf), use & 1u, abort_flag)) {
                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_EPILOGUE); *abort_flag = 1; ok = false; break;
            }
            BLZ_T_ADD(t_wait, tw);
            [[maybe_unused]] const long long te = BLZ_T_NOW();
            tc_fence_after_sync();
            const int row = m_tile * 128 + q * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t acc[32];
                tmem_ld32(t_row + c0, acc);
                tmem_ld_wait();
                epilogue_store32_dyn(p.epi, acc, row, n_tile * BN + c0, p.M, p.N);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(buf));
            BLZ_T_ADD(t_work, te);
        }
        BLZ_T_ADD(t_total, t_begin);
        if (warp == 4 && lane == 0) { BLZ_T_STORE(5, t_wait); BLZ_T_STORE(6, t_work); BLZ_T_STORE(7, t_total); }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        // Error path only: give TMA copies still in flight time to land before the CTA retires.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace blz
