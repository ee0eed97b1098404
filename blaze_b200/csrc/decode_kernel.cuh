// decode_kernel.cuh -- NVFP4 GEMM for skinny activations (M <= 64): HBM-bound weight streaming.
//
//   C[M,N] = epilogue( alpha * sum_k X[M,K] * W[N,K]^T )
//
// The operands are swapped with respect to the tiled kernel: 128 weight rows fill the 128-row
// side of the tensor-core instruction and the M activation rows are its N (16, 32 or 64), so no
// tensor work is spent on padding (Blaze pads M to a 128-row tile:
// src/kernels/gemm_fp4_blkscaled_sm100.cu:883-890).  K is split across CTAs so that every SM
// streams weights; each split writes fp32 partial sums and the CTA that arrives last at a tile
// adds them in split order 0..S-1, which keeps the result independent of arrival order.
//
// Warp roles as in gemm_cluster_kernel.cuh: warp 0 TMA producer, warp 1 MMA issuer, warp 2 tensor-memory
// allocation, warps 4-7 epilogue.  Two CTAs fit one SM.
#pragma once

#include "common.cuh"

namespace blz {

struct DecodeKernelParams {
    int M, N;
    int n_tiles;             // ceil(N / 128)
    int k_stages_total;      // ceil(K/2 bytes / 128)
    int stages_per_split;
    int split;
    uint32_t idesc;
    const uint8_t* sfw;      // tiled scale factors of the weights  [row blocks][sf_katoms][512]
    const uint8_t* sfx;      // tiled scale factors of the activations (row block 0 is used)
    int sf_katoms;
    float* partial;          // [split][MMA_N][n_tiles*128] fp32, only when split > 1
    int* counters;           // [n_tiles], zero between launches
    EpilogueParams epi;
    int* status;
};

__device__ __forceinline__ void epilogue_store_one(const EpilogueParams& e, float acc, int m, int n) {
    float v = acc * e.alpha;
    if ((e.mode == EPI_BIAS || e.mode == EPI_BIAS_SILU) && e.bias != nullptr) {
        v += e.out_type == OUT_BF16 ? load_out_elem<OUT_BF16>(e.bias, n) : e.out_type == OUT_F16 ? load_out_elem<OUT_F16>(e.bias, n) : load_out_elem<OUT_F32>(e.bias, n);
    }
    if (e.mode == EPI_SILU || e.mode == EPI_BIAS_SILU) v = silu_f32(v);
    const long long off = static_cast<long long>(m) * e.ldc + n;
    if (e.mode == EPI_RESIDUAL && e.residual != nullptr) {
        const long long roff = static_cast<long long>(m) * e.ldr + n;
        v += e.out_type == OUT_BF16 ? load_out_elem<OUT_BF16>(e.residual, roff) : e.out_type == OUT_F16 ? load_out_elem<OUT_F16>(e.residual, roff) : load_out_elem<OUT_F32>(e.residual, roff);
    }
    if (e.out_type == OUT_BF16) reinterpret_cast<__nv_bfloat16*>(e.C)[off] = __float2bfloat16_rn(v);
    else if (e.out_type == OUT_F16) reinterpret_cast<__half*>(e.C)[off] = __float2half_rn(clamp_f16_range(v));
    else reinterpret_cast<float*>(e.C)[off] = v;
}

template <int MMA_N, int STAGES>
struct DecodeConfig {
    static constexpr uint32_t W_BYTES = 128 * 128;
    static constexpr uint32_t X_BYTES = MMA_N * 128;
    static constexpr uint32_t X_REGION = X_BYTES < 1024 ? 1024 : X_BYTES;   // keeps every tile 1024-byte aligned
    static constexpr uint32_t SF_BYTES = 4 * 512;
    static constexpr uint32_t STAGE_BYTES = W_BYTES + X_REGION + 2 * SF_BYTES;
    static constexpr uint32_t TX_BYTES = W_BYTES + X_BYTES + 2 * SF_BYTES;
    static constexpr uint32_t SFW_COL = 64, SFX_COL = 80, TMEM_COLS = 128;
    static constexpr uint32_t BAR_BYTES = 8 * (2 * STAGES + 1) + 16;
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
    static_assert(MMA_N % 16 == 0 && MMA_N >= 16 && MMA_N <= 64, "activation rows per instruction");
    static_assert(SMEM_BYTES <= 115000, "two CTAs must fit one SM");
};

template <int MMA_N, int STAGES>
__global__ void __launch_bounds__(256, 2)
decode_nvf4_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const DecodeKernelParams p) {
    using Cfg = DecodeConfig<MMA_N, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - raw);

    const uint32_t bar_base = base + STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * STAGES);
    const uint32_t slot_off = STAGES * Cfg::STAGE_BYTES + 8u * (2 * STAGES + 1);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + slot_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + slot_off + 4);
    volatile int* ticket_slot = reinterpret_cast<volatile int*>(gen_base + slot_off + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    [[maybe_unused]] const long long t_entry = BLZ_T_NOW();
    BLZ_T_STORE_IF(threadIdx.x == 0, 9, global_timer_ns());
    const int n_tile = blockIdx.x % p.n_tiles, split_idx = blockIdx.x / p.n_tiles;
    const int ks_begin = split_idx * p.stages_per_split;
    const int ks_end = min(p.k_stages_total, ks_begin + p.stages_per_split);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(acc_full_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 2) {
        tmem_alloc(base + slot_off, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&tm_w);
        prefetch_tensormap(&tm_x);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    BLZ_T_STORE_IF(threadIdx.x == 0, 11, clock64() - t_entry);   // set-up

    if (warp == 0) {
        if (elect_one()) {
            BLZ_T_DECL(t_wait);
            const uint64_t pol_stream = l2_policy_evict_first();   // weights are read once
            const uint64_t pol_keep = l2_policy_evict_last();      // activations are shared by every CTA
            int stage = 0; uint32_t phase = 0;
            for (int ks = ks_begin; ks < ks_end; ++ks) {
                [[maybe_unused]] const long long tw = BLZ_T_NOW();
                if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; break;
                }
                BLZ_T_ADD(t_wait, tw);
                const uint32_t sw = base + stage * Cfg::STAGE_BYTES;
                const uint32_t sx = sw + Cfg::W_BYTES;
                const uint32_t ssfw = sx + Cfg::X_REGION;
                const uint32_t ssfx = ssfw + Cfg::SF_BYTES;
                mbar_arrive_expect_tx(full_bar(stage), Cfg::TX_BYTES);
                tma_load_2d_hint(sw, &tm_w, ks * 128, n_tile * 128, full_bar(stage), pol_stream);
                tma_load_2d_hint(sx, &tm_x, ks * 128, 0, full_bar(stage), pol_keep);
                const size_t katom = static_cast<size_t>(ks) * 4;
                bulk_load_1d(ssfw, p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + katom) * 512, Cfg::SF_BYTES, full_bar(stage));
                bulk_load_1d(ssfx, p.sfx + katom * 512, Cfg::SF_BYTES, full_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            BLZ_T_STORE(0, t_wait); BLZ_T_STORE(1, BLZ_T_NOW() - t_entry);
        }
        __syncwarp();
    } else if (warp == 1) {
        if (elect_one()) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            BLZ_T_DECL(t_wait_full);
            for (int ks = ks_begin; ks < ks_end; ++ks) {
                [[maybe_unused]] const long long tf = BLZ_T_NOW();
                if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                }
                BLZ_T_ADD(t_wait_full, tf);
                BLZ_T_STORE_IF(ks == ks_begin, 12, clock64() - t_entry);   // first stage landed
                tc_fence_after_sync();
                const uint32_t sw = base + stage * Cfg::STAGE_BYTES;
                const uint32_t sx = sw + Cfg::W_BYTES;
                const uint32_t ssfw = sx + Cfg::X_REGION;
                const uint32_t ssfx = ssfw + Cfg::SF_BYTES;
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    tc_copy_sf(tmem_base + Cfg::SFW_COL + 4 * a, make_desc_sf(ssfw + a * 512));
                    tc_copy_sf(tmem_base + Cfg::SFX_COL + 4 * a, make_desc_sf(ssfx + a * 512));
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t accumulate = (ks != ks_begin || k != 0) ? 1u : 0u;
                    umma_nvf4(tmem_base, make_desc_k_sw128(sw + k * 32), make_desc_k_sw128(sx + k * 32), p.idesc,
                              tmem_base + Cfg::SFW_COL + 4 * k, tmem_base + Cfg::SFX_COL + 4 * k, accumulate);
                }
                tc_commit(empty_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) tc_commit(acc_full_bar);
            BLZ_T_STORE(2, t_wait_full); BLZ_T_STORE(4, BLZ_T_NOW() - t_entry);
        }
        __syncwarp();
    } else if (warp >= 4) {
        const int q = warp & 3;
        const int epi_tid = threadIdx.x - 128;
        // Every epilogue thread walks the same barrier sequence below whether or not its wait
        // succeeded, so a give-up in one warp can never strand the others at a named barrier.
        const bool ok = mbar_wait(acc_full_bar, 0u, abort_flag);
        BLZ_T_STORE_IF(threadIdx.x == 128, 5, clock64() - t_entry);       // accumulator finished
        if (!ok) { atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_EPILOGUE); *abort_flag = 1; }
        float acc[MMA_N];
#pragma unroll
        for (int m = 0; m < MMA_N; ++m) acc[m] = 0.0f;
        if (ok) {
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
            for (int c = 0; c < MMA_N; c += 16) {
                uint32_t r[16];
                tmem_ld16(t_row + c, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c + j] = __uint_as_float(r[j]);
            }
            tc_fence_before_sync();
        }
        const int n = n_tile * 128 + q * 32 + lane;
        if (p.split == 1) {
            if (ok && n < p.N) {
#pragma unroll
                for (int m = 0; m < MMA_N; ++m)
                    if (m < p.M) epilogue_store_one(p.epi, acc[m], m, n);
            }
        } else {
            const long long npad = static_cast<long long>(p.n_tiles) * 128;
            float* mine = p.partial + static_cast<long long>(split_idx) * MMA_N * npad + n;
#pragma unroll
            for (int m = 0; m < MMA_N; ++m)
                if (m < p.M) __stcg(mine + m * npad, acc[m]);
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (epi_tid == 0) *ticket_slot = atomicAdd(p.counters + n_tile, 1);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*ticket_slot == p.split - 1) {
                // Last split to arrive at this tile: add the partial sums in split order.
                __threadfence();
                if (n < p.N) {
                    for (int m = 0; m < p.M; ++m) {
                        float sum = 0.0f;
                        for (int s = 0; s < p.split; ++s)
                            sum += __ldcg(p.partial + (static_cast<long long>(s) * MMA_N + m) * npad + n);
                        epilogue_store_one(p.epi, sum, m, n);
                    }
                }
                if (epi_tid == 0) p.counters[n_tile] = 0;
            }
        }
    }

    BLZ_T_STORE_IF(threadIdx.x == 128, 7, clock64() - t_entry);           // epilogue finished
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
    BLZ_T_STORE_IF(threadIdx.x == 0, 10, global_timer_ns()); BLZ_T_STORE_IF(threadIdx.x == 0, 8, clock64() - t_entry);
}

}  // namespace blz
