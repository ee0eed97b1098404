// decode_stream_kernel.cuh -- NVFP4 GEMM for skinny activations (M <= 64), second generation:
// an HBM-bound weight stream with every fixed cost taken off the critical path.
//
//   C[M,N] = epilogue( alpha * sum_k X[M,K] * W[N,K]^T )
//
// As in decode_kernel.cuh the operands are swapped (128 weight rows are the instruction's M, the
// activations its N) and K is split so that every SM streams weights.  What differs:
//   - a K split is a thread-block cluster: the S CTAs of a tile reduce their fp32 partial sums
//     through distributed shared memory (non-leaders store into the leader's stage buffers, the
//     leader adds them in split order 0..S-1), so there is no global scratch, no atomic, no
//     __threadfence, and the result is still independent of arrival order;
//   - scale factors reach tensor memory through tcgen05.st from four helper warps into per-stage
//     columns, so the tensor pipe only sees four MMAs per stage (a tcgen05.cp costs ~70 cycles of
//     that pipe each, eight per stage before);
//   - programmatic dependent launch: the kernel lets its successor start early and itself
//     prefetches its first weight stages (which no earlier kernel produces) before waiting for its
//     predecessor; only the activation loads and everything after them wait;
//   - the epilogue transposes through shared memory and writes C rows with 16-byte stores.
//
// Warps: 0 TMA producer, 1 MMA issuer, 2 tensor-memory alloc, 4-7 epilogue, 8-11 scale factors.
#pragma once

#include "common.cuh"

namespace blz {

struct DecodeStreamParams {
    int M, N;
    int n_tiles;             // ceil(N / 128)
    int k_stages_total;      // ceil(K/2 bytes / 128)
    int stages_per_split;
    int split;               // = cluster size: 1, 2, 4 or 8
    uint32_t idesc;
    const uint8_t* sfw;      // tiled scale factors of the weights
    const uint8_t* sfx;      // tiled scale factors of the activations (row block 0)
    int sf_katoms;
    EpilogueParams epi;
    int* status;
};

__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// store a float into the shared memory of CTA `cta` of this cluster at the same offset as `addr`
__device__ __forceinline__ void st_shared_cluster_f32(uint32_t addr, uint32_t cta, float v) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "st.shared::cluster.f32 [ra], %2;\n\t}"
        ::"r"(addr), "r"(cta), "f"(v) : "memory");
}

template <int MMA_N, int STAGES>
struct DecodeStreamConfig {
    static constexpr uint32_t W_BYTES = 128 * 128;
    static constexpr uint32_t X_BYTES = MMA_N * 128;
    static constexpr uint32_t X_REGION = X_BYTES < 1024 ? 1024 : X_BYTES;
    static constexpr uint32_t SF_BYTES = 4 * 512;
    static constexpr uint32_t STAGE_BYTES = W_BYTES + X_REGION + 2 * SF_BYTES;
    static constexpr uint32_t TX_BYTES = W_BYTES + X_BYTES + 2 * SF_BYTES;
    static constexpr uint32_t SF_COLS = 32;                 // per stage: weights 16, activations 16
    static constexpr uint32_t SF_BASE = 64;                 // accumulator in columns [0, MMA_N)
    static constexpr uint32_t TMEM_COLS = 256;
    static constexpr uint32_t NUM_BARS = 3 * STAGES + 1;
    static constexpr uint32_t BAR_BYTES = 8 * NUM_BARS + 16;
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
    static constexpr int MAX_SPLIT = (STAGES * STAGE_BYTES) / (MMA_N * 128 * 4) + 1 < 8 ? (STAGES * STAGE_BYTES) / (MMA_N * 128 * 4) + 1 : 8;
    static_assert(MMA_N % 16 == 0 && MMA_N >= 16 && MMA_N <= 64, "activation rows per instruction");
    static_assert(SF_BASE + STAGES * SF_COLS <= TMEM_COLS, "scale-factor columns exceed the allocation");
    static_assert(SMEM_BYTES <= 115000, "two CTAs must fit one SM");
    static_assert(MMA_N * 128 * 4 <= STAGES * STAGE_BYTES, "output staging must fit the stage buffers");
};

template <int MMA_N, int STAGES>
__global__ void __launch_bounds__(384, (MMA_N <= 32 ? 2 : 1))
decode_stream_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const DecodeStreamParams p) {
    using Cfg = DecodeStreamConfig<MMA_N, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - raw);

    const uint32_t bar_base = base + STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto ready_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (3 * STAGES);
    const uint32_t slot_off = STAGES * Cfg::STAGE_BYTES + 8u * Cfg::NUM_BARS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + slot_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + slot_off + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tile = blockIdx.x / p.split;
    const int split_idx = blockIdx.x % p.split;             // = rank in the cluster
    const int ks_begin = split_idx * p.stages_per_split;
    const int ks_end = min(p.k_stages_total, ks_begin + p.stages_per_split);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(ready_bar(s), 4); mbar_init(empty_bar(s), 1); }
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
    // Everything this grid still needs from its predecessor is read after griddep_wait(); the
    // successor may start its own set-up and weight prefetch now.
    griddep_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol_stream = l2_policy_evict_first();   // weights are read once
            const uint64_t pol_keep = l2_policy_evict_last();      // activations are shared by every CTA
            int stage = 0; uint32_t phase = 0;
            // weights and their scales of the first ring of stages do not depend on earlier kernels
            const int n_pre = min(ks_end - ks_begin, STAGES);
            for (int i = 0; i < n_pre; ++i) {
                const int ks = ks_begin + i;
                const uint32_t sw = base + i * Cfg::STAGE_BYTES;
                const uint32_t ssfw = sw + Cfg::W_BYTES + Cfg::X_REGION;
                mbar_arrive_expect_tx(full_bar(i), Cfg::TX_BYTES);
                tma_load_2d_hint(sw, &tm_w, ks * 128, n_tile * 128, full_bar(i), pol_stream);
                bulk_load_1d(ssfw, p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + static_cast<size_t>(ks) * 4) * 512, Cfg::SF_BYTES, full_bar(i));
            }
            griddep_wait();
            for (int ks = ks_begin; ks < ks_end; ++ks) {
                const uint32_t sw = base + stage * Cfg::STAGE_BYTES;
                const uint32_t sx = sw + Cfg::W_BYTES;
                const uint32_t ssfw = sx + Cfg::X_REGION;
                const uint32_t ssfx = ssfw + Cfg::SF_BYTES;
                const size_t katom = static_cast<size_t>(ks) * 4;
                if (ks - ks_begin >= STAGES) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; break;
                    }
                    mbar_arrive_expect_tx(full_bar(stage), Cfg::TX_BYTES);
                    tma_load_2d_hint(sw, &tm_w, ks * 128, n_tile * 128, full_bar(stage), pol_stream);
                    bulk_load_1d(ssfw, p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + katom) * 512, Cfg::SF_BYTES, full_bar(stage));
                }
                tma_load_2d_hint(sx, &tm_x, ks * 128, 0, full_bar(stage), pol_keep);
                bulk_load_1d(ssfx, p.sfx + katom * 512, Cfg::SF_BYTES, full_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int ks = ks_begin; ks < ks_end; ++ks) {
                if (!mbar_wait(ready_bar(stage), phase, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                }
                tc_fence_after_sync();
                const uint32_t sw = base + stage * Cfg::STAGE_BYTES;
                const uint32_t sx = sw + Cfg::W_BYTES;
                const uint32_t sf_cols = tmem_base + Cfg::SF_BASE + stage * Cfg::SF_COLS;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t accumulate = (ks != ks_begin || k != 0) ? 1u : 0u;
                    umma_nvf4(tmem_base, make_desc_k_sw128(sw + k * 32), make_desc_k_sw128(sx + k * 32), p.idesc,
                              sf_cols + 4 * k, sf_cols + 16 + 4 * k, accumulate);
                }
                tc_commit(empty_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) tc_commit(acc_full_bar);
        }
        __syncwarp();
    } else if (warp >= 8) {
        // scale factors: shared memory -> registers -> this stage's tensor-memory columns
        const int q = warp & 3;
        int stage = 0; uint32_t phase = 0;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; break;
            }
            const uint8_t* ssfw = gen_base + stage * Cfg::STAGE_BYTES + Cfg::W_BYTES + Cfg::X_REGION;
            const uint8_t* ssfx = ssfw + Cfg::SF_BYTES;
            const uint32_t t_sf = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::SF_BASE + stage * Cfg::SF_COLS;
            uint32_t r[32];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const uint4 v = *reinterpret_cast<const uint4*>(ssfw + a * 512 + lane * 16);
                r[4 * a] = v.x; r[4 * a + 1] = v.y; r[4 * a + 2] = v.z; r[4 * a + 3] = v.w;
                const uint4 u = *reinterpret_cast<const uint4*>(ssfx + a * 512 + lane * 16);
                r[16 + 4 * a] = u.x; r[16 + 4 * a + 1] = u.y; r[16 + 4 * a + 2] = u.z; r[16 + 4 * a + 3] = u.w;
            }
            tmem_st32(t_sf, r);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(ready_bar(stage));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
    }

    // ------------------------------------------------------------------ epilogue
    // Epilogue warps wait for the accumulator; with a K split every thread of every CTA of the
    // cluster then meets at two cluster barriers (reached on every path, also after a give-up).
    float acc[MMA_N];
    bool epi_ok = true;
    const bool is_epi = (warp >= 4 && warp < 8);
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    if (is_epi) {
        epi_ok = mbar_wait(acc_full_bar, 0u, abort_flag);
        if (!epi_ok) { atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_EPILOGUE); *abort_flag = 1; }
#pragma unroll
        for (int m = 0; m < MMA_N; ++m) acc[m] = 0.0f;
        if (epi_ok) {
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
            for (int c = 0; c < MMA_N; c += 16) {
                uint32_t r[16];
                tmem_ld16(t_row + c, r);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c + j] = __uint_as_float(r[j]);
            }
            tmem_ld_wait();
            tc_fence_before_sync();
        }
    }
    if (p.split > 1) {
        cluster_sync_all();                 // every CTA of the tile is past its main loop: the leader's stage buffers are free
        if (is_epi && split_idx != 0) {
            // partial sums of split s go to slot s-1 of the leader: [slot][m][128] fp32
            const uint32_t dst = base + (static_cast<uint32_t>(split_idx - 1) * MMA_N * 128 + n_local) * 4;
#pragma unroll
            for (int m = 0; m < MMA_N; ++m)
                if (m < p.M) st_shared_cluster_f32(dst + m * 512, 0, acc[m]);
        }
        cluster_sync_all();                 // partial sums have landed in the leader
        if (is_epi && split_idx == 0) {
            const float* part = reinterpret_cast<const float*>(gen_base);
#pragma unroll
            for (int m = 0; m < MMA_N; ++m) {
                if (m < p.M) {
                    float sum = acc[m];
                    for (int s = 1; s < p.split; ++s) sum += part[(s - 1) * MMA_N * 128 + m * 128 + n_local];
                    acc[m] = sum;
                }
            }
        }
    }
    if (is_epi && split_idx == 0) {
        // transpose through shared memory ([m][128] in the output type), then row-wise 16-byte stores
        const EpilogueParams& e = p.epi;
        const int esize = e.out_type == OUT_F32 ? 4 : 2;
        const int n = n_tile * 128 + n_local;
        griddep_wait();                      // bias / residual may come from the predecessor; C may be read by it
        named_barrier_sync(1, 128);          // all reads of the partial sums are done: the buffer can be reused
        uint8_t* stag = gen_base;
#pragma unroll
        for (int m = 0; m < MMA_N; ++m) {
            if (m < p.M) {
                float v = acc[m] * e.alpha;
                if (n < p.N) {
                    if ((e.mode == EPI_BIAS || e.mode == EPI_BIAS_SILU) && e.bias != nullptr)
                        v += e.out_type == OUT_BF16 ? load_out_elem<OUT_BF16>(e.bias, n) : e.out_type == OUT_F16 ? load_out_elem<OUT_F16>(e.bias, n) : load_out_elem<OUT_F32>(e.bias, n);
                    if (e.mode == EPI_SILU || e.mode == EPI_BIAS_SILU) v = silu_f32(v);
                    if (e.mode == EPI_RESIDUAL && e.residual != nullptr) {
                        const long long roff = static_cast<long long>(m) * e.ldr + n;
                        v += e.out_type == OUT_BF16 ? load_out_elem<OUT_BF16>(e.residual, roff) : e.out_type == OUT_F16 ? load_out_elem<OUT_F16>(e.residual, roff) : load_out_elem<OUT_F32>(e.residual, roff);
                    }
                }
                if (e.out_type == OUT_F32) reinterpret_cast<float*>(stag)[m * 128 + n_local] = v;
                else if (e.out_type == OUT_BF16) reinterpret_cast<__nv_bfloat16*>(stag)[m * 128 + n_local] = __float2bfloat16_rn(v);
                else reinterpret_cast<__half*>(stag)[m * 128 + n_local] = __float2half_rn(clamp_f16_range(v));
            }
        }
        named_barrier_sync(1, 128);
        if (epi_ok) {
            const int row_bytes = 128 * esize;
            const int chunks_per_row = row_bytes / 16;
            const int tid = threadIdx.x - 128;
            const int cols_per_chunk = 16 / esize;
            for (int c = tid; c < p.M * chunks_per_row; c += 128) {
                const int m = c / chunks_per_row, j = c % chunks_per_row;
                const int col = n_tile * 128 + j * cols_per_chunk;
                if (col >= p.N) continue;
                uint8_t* dst = reinterpret_cast<uint8_t*>(e.C) + (static_cast<long long>(m) * e.ldc + col) * esize;
                const uint8_t* src = stag + m * row_bytes + j * 16;
                if (e.vec_ok && col + cols_per_chunk <= p.N) {
                    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
                } else {
                    for (int b = 0; b < 16 && col * esize + b < p.N * esize; ++b) dst[b] = src[b];
                }
            }
        }
    }

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
}

}  // namespace blz
