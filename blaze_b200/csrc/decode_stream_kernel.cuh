// decode_stream_kernel.cuh -- GEMM for skinny activations (M <= 64): an HBM-bound weight stream
// with every fixed cost taken off the critical path.  decode_stream_kernel covers NVFP4, FP8 and
// the dense 16-bit kinds (operands reach shared memory ready for the tensor core);
// decode_w4a16_kernel covers 16-bit activations times NVFP4 weights (helper warps expand the
// packed weights into the 16-bit operand tile on the way).
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
// Warps: 0 TMA producer, 1 MMA issuer, 2 tensor-memory alloc, 4-7 epilogue, 8-11 scale factors
// (NVFP4 only; the other kinds run 8 warps).
#pragma once

#include "common.cuh"

namespace blz {

struct DecodeStreamParams {
    int M, N;
    int n_tiles;             // ceil(N / 128)
    int k_stages_total;      // ceil(bytes of one operand row / 128); W4A16: ceil(K / 64)
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

// Shared by both kernels, called by every thread of the CTA once its main-loop role is done.
// Warps 4-7 take the fp32 sums out of tensor memory (columns [0, MMA_N), lane = weight row); with
// a K split every thread of every CTA of the cluster meets at two cluster barriers around the
// reduction through the leader's shared memory (at `base`, free once the main loops are over);
// the leader applies the epilogue and writes C.
template <int MMA_N>
__device__ __forceinline__ void decode_epilogue(const DecodeStreamParams& p, uint32_t base, uint8_t* gen_base, uint32_t tmem_base,
                                                uint32_t acc_full_bar, volatile int* abort_flag, int n_tile, int split_idx,
                                                int warp, int lane, [[maybe_unused]] long long t_entry) {
    // Epilogue warps wait for the accumulator; with a K split every thread of every CTA of the
    // cluster then meets at two cluster barriers (reached on every path, also after a give-up).
    float acc[MMA_N];
    bool epi_ok = true;
    const bool is_epi = (warp >= 4 && warp < 8);
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    // The epilogue's parameters are fetched now, while these warps would only wait: the first touch
    // of a parameter line costs a constant-cache miss of several hundred cycles, and this kernel's
    // epilogue runs once, on the critical path of the next kernel in the stream.
    const float e_alpha = p.epi.alpha;
    const int e_mode = p.epi.mode, e_out = p.epi.out_type, e_vec = p.epi.vec_ok, p_M = p.M, p_N = p.N, p_split = p.split;
    const long long e_ldc = p.epi.ldc, e_ldr = p.epi.ldr;
    void* const e_C = p.epi.C;
    const void* const e_bias = p.epi.bias;
    const void* const e_res = p.epi.residual;
    asm volatile("" ::"f"(e_alpha), "r"(e_mode), "r"(e_out), "r"(e_vec), "r"(p_M), "r"(p_N), "r"(p_split), "l"(e_ldc), "l"(e_ldr), "l"(e_C), "l"(e_bias), "l"(e_res));
    if (is_epi) {
        epi_ok = mbar_wait(acc_full_bar, 0u, abort_flag);
#ifdef BLZ_KERNEL_TIMING
        if (threadIdx.x == 128) BLZ_T_STORE(5, clock64() - t_entry);
#endif
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
#ifdef BLZ_KERNEL_TIMING
        if (threadIdx.x == 128) BLZ_T_STORE(1, clock64() - t_entry);
#endif
    }
    if (p_split > 1) {
        cluster_sync_all();                 // every CTA of the tile is past its main loop: the leader's stage buffers are free
        if (is_epi && split_idx != 0) {
            // partial sums of split s go to slot s-1 of the leader: [slot][m][128] fp32
            const uint32_t dst = base + (static_cast<uint32_t>(split_idx - 1) * MMA_N * 128 + n_local) * 4;
#pragma unroll
            for (int m = 0; m < MMA_N; ++m)
                if (m < p_M) st_shared_cluster_f32(dst + m * 512, 0, acc[m]);
        }
        cluster_sync_all();                 // partial sums have landed in the leader
        if (is_epi && split_idx == 0) {
            const float* part = reinterpret_cast<const float*>(gen_base);
#pragma unroll
            for (int m = 0; m < MMA_N; ++m) {
                if (m < p_M) {
                    float sum = acc[m];
                    for (int s = 1; s < p_split; ++s) sum += part[(s - 1) * MMA_N * 128 + m * 128 + n_local];
                    acc[m] = sum;
                }
            }
        }
    }
    if (is_epi && split_idx == 0) {
        // Transpose through shared memory: the raw fp32 sums go to [m][128] with the shortest
        // possible straight-line code (this code runs once per CTA, so every instruction line is an
        // instruction-cache miss on the critical path); the epilogue arithmetic and the narrowing
        // happen in the compact row-store loop below.
#ifdef BLZ_KERNEL_TIMING
        if (threadIdx.x == 128) BLZ_T_STORE(2, clock64() - t_entry);
#endif
        griddep_wait();                      // bias / residual may come from the predecessor; C may be read by it
        named_barrier_sync(1, 128);          // all reads of the partial sums are done: the buffer can be reused
        float* stag = reinterpret_cast<float*>(gen_base);
#pragma unroll
        for (int m = 0; m < MMA_N; ++m) stag[m * 128 + n_local] = acc[m];
        named_barrier_sync(1, 128);
#ifdef BLZ_KERNEL_TIMING
        if (threadIdx.x == 128) BLZ_T_STORE(6, clock64() - t_entry);
#endif
        if (epi_ok) {
            const int tid = threadIdx.x - 128;
            const int esize = e_out == OUT_F32 ? 4 : 2;
            // one item = 8 consecutive columns of one row: 128 / 8 = 16 items per row
#pragma unroll 1
            for (int c = tid; c < p_M * 16; c += 128) {
                const int m = c >> 4, j = c & 15;
                const int col = n_tile * 128 + j * 8;
                if (col >= p_N) continue;
                const float4 lo = *reinterpret_cast<const float4*>(stag + m * 128 + j * 8);
                const float4 hi = *reinterpret_cast<const float4*>(stag + m * 128 + j * 8 + 4);
                float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int t = 0; t < 8; ++t) v[t] *= e_alpha;
                if (e_mode != EPI_NONE) {
#pragma unroll 1
                    for (int t = 0; t < 8; ++t) {
                        const int n = col + t;
                        if (n >= p_N) break;
                        if ((e_mode == EPI_BIAS || e_mode == EPI_BIAS_SILU) && e_bias != nullptr)
                            v[t] += e_out == OUT_BF16 ? load_out_elem<OUT_BF16>(e_bias, n) : e_out == OUT_F16 ? load_out_elem<OUT_F16>(e_bias, n) : load_out_elem<OUT_F32>(e_bias, n);
                        if (e_mode == EPI_SILU || e_mode == EPI_BIAS_SILU) v[t] = silu_f32(v[t]);
                        if (e_mode == EPI_RESIDUAL && e_res != nullptr) {
                            const long long roff = static_cast<long long>(m) * e_ldr + n;
                            v[t] += e_out == OUT_BF16 ? load_out_elem<OUT_BF16>(e_res, roff) : e_out == OUT_F16 ? load_out_elem<OUT_F16>(e_res, roff) : load_out_elem<OUT_F32>(e_res, roff);
                        }
                    }
                }
                uint8_t* dst = reinterpret_cast<uint8_t*>(e_C) + (static_cast<long long>(m) * e_ldc + col) * esize;
                const bool whole = e_vec && col + 8 <= p_N;
                if (e_out == OUT_F32) {
                    if (whole) {
                        reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
                        reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
                    } else {
                        for (int t = 0; t < 8 && col + t < p_N; ++t) reinterpret_cast<float*>(dst)[t] = v[t];
                    }
                } else {
                    uint32_t w[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) w[t] = pack2_out(e_out, v[2 * t], v[2 * t + 1]);
                    if (whole) {
                        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                    } else {
                        for (int t = 0; t < 8 && col + t < p_N; ++t)
                            reinterpret_cast<uint16_t*>(dst)[t] = static_cast<uint16_t>(w[t >> 1] >> (16 * (t & 1)));
                    }
                }
            }
        }
    }

#ifdef BLZ_KERNEL_TIMING
    if (threadIdx.x == 128) BLZ_T_STORE(7, clock64() - t_entry);
#endif
}

// Every thread of the CTA: after a give-up let copies in flight land, then free tensor memory.
__device__ __forceinline__ void decode_teardown(uint32_t tmem_base, uint32_t tmem_cols, volatile int* abort_flag, int warp) {
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, tmem_cols);
    }
#ifdef BLZ_KERNEL_TIMING
    if (threadIdx.x == 0) { BLZ_T_STORE(10, global_timer_ns()); }
#endif
}

template <int KIND, int MMA_N, int STAGES>
struct DecodeStreamConfig {
    static constexpr bool HAS_SF = (KIND == MMA_NVF4);
    static constexpr int THREADS = HAS_SF ? 384 : 256;
    static constexpr uint32_t W_BYTES = 128 * 128;
    static constexpr uint32_t X_BYTES = MMA_N * 128;
    static constexpr uint32_t X_REGION = X_BYTES < 1024 ? 1024 : X_BYTES;
    static constexpr uint32_t SF_BYTES = HAS_SF ? 4 * 512 : 0;
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
    static_assert(!HAS_SF || SF_BASE + STAGES * SF_COLS <= TMEM_COLS, "scale-factor columns exceed the allocation");
    static_assert(SMEM_BYTES <= 115000, "two CTAs must fit one SM");
    static_assert(MMA_N * 128 * 4 <= STAGES * STAGE_BYTES, "fp32 output staging must fit the stage buffers");
};

template <int KIND, int MMA_N, int STAGES>
__global__ void __launch_bounds__((DecodeStreamConfig<KIND, MMA_N, STAGES>::THREADS), (MMA_N <= 32 ? 2 : 1))
decode_stream_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const DecodeStreamParams p) {
    using Cfg = DecodeStreamConfig<KIND, MMA_N, STAGES>;
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
    [[maybe_unused]] const long long t_entry = BLZ_T_NOW();
#ifdef BLZ_KERNEL_TIMING
    if (threadIdx.x == 0) BLZ_T_STORE(9, global_timer_ns());
#endif
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
#ifndef BLZ_DECODE_LATE_DEPENDENTS
    // Everything this grid still needs from its predecessor is read after griddep_wait(); the
    // successor may start its own set-up and weight prefetch now.
    griddep_launch_dependents();
#endif
#ifdef BLZ_KERNEL_TIMING
    if (threadIdx.x == 0) BLZ_T_STORE(11, clock64() - t_entry);
#endif

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
                if constexpr (Cfg::HAS_SF)
                    bulk_load_1d(ssfw, p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + static_cast<size_t>(ks) * 4) * 512, Cfg::SF_BYTES, full_bar(i));
            }
            griddep_wait();
#ifdef BLZ_DECODE_LATE_DEPENDENTS
            griddep_launch_dependents();     // at most one successor prefetches while this grid runs
#endif
#ifdef BLZ_KERNEL_TIMING
            BLZ_T_STORE(12, clock64() - t_entry); BLZ_T_STORE(14, global_timer_ns());
#endif
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
                    if constexpr (Cfg::HAS_SF)
                        bulk_load_1d(ssfw, p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + katom) * 512, Cfg::SF_BYTES, full_bar(stage));
                }
                tma_load_2d_hint(sx, &tm_x, ks * 128, 0, full_bar(stage), pol_keep);
                if constexpr (Cfg::HAS_SF) bulk_load_1d(ssfx, p.sfx + katom * 512, Cfg::SF_BYTES, full_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int ks = ks_begin; ks < ks_end; ++ks) {
                // without scale factors nothing stands between "landed" and "ready"
                if (!mbar_wait(Cfg::HAS_SF ? ready_bar(stage) : full_bar(stage), phase, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                }
#ifdef BLZ_KERNEL_TIMING
                if (ks == ks_begin) BLZ_T_STORE(13, clock64() - t_entry);
#endif
                tc_fence_after_sync();
                const uint32_t sw = base + stage * Cfg::STAGE_BYTES;
                const uint32_t sx = sw + Cfg::W_BYTES;
                [[maybe_unused]] const uint32_t sf_cols = tmem_base + Cfg::SF_BASE + stage * Cfg::SF_COLS;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t accumulate = (ks != ks_begin || k != 0) ? 1u : 0u;
                    const uint64_t wd = make_desc_k_sw128(sw + k * 32), xd = make_desc_k_sw128(sx + k * 32);
                    if constexpr (KIND == MMA_F16) umma_f16(tmem_base, wd, xd, p.idesc, accumulate);
                    else if constexpr (KIND == MMA_F8) umma_f8(tmem_base, wd, xd, p.idesc, accumulate);
                    else umma_nvf4(tmem_base, wd, xd, p.idesc, sf_cols + 4 * k, sf_cols + 16 + 4 * k, accumulate);
                }
                tc_commit(empty_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) tc_commit(acc_full_bar);
            BLZ_T_STORE(4, BLZ_T_NOW() - t_entry);
        }
        __syncwarp();
    } else if (Cfg::HAS_SF && warp >= 8) {
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

    decode_epilogue<MMA_N>(p, base, gen_base, tmem_base, acc_full_bar, abort_flag, n_tile, split_idx, warp, lane, t_entry);
    decode_teardown(tmem_base, Cfg::TMEM_COLS, abort_flag, warp);
}

// ------------------------------------------------------------------------------------------------
// 16-bit activations x NVFP4 weights.
//
// The tensor core has no instruction that takes one 4-bit and one 16-bit operand, so the packed
// weights are expanded on the way: eight helper warps turn every stage of packed weights (128 rows
// x 64 K values = 4 KB, plus one 512-byte atom of block scales) into the fp16 operand tile
// in the activations' 16-bit format (q * block scale: at most six significant bits, exact in fp16
// and in bf16), 128-byte swizzled like a TMA load would have left it.  Both operands of a
// kind::f16 instruction must have the same format -- an fp16 A with a bf16 B is rejected by the
// hardware as an illegal instruction -- so bf16 activations need bf16 weights, which cost three
// more integer instructions per pair of values than fp16 (there is no E2M1 -> bf16 conversion).
// HBM only ever sees the 4.5 bits per weight.
//
// Two rings: a deep one of small load stages (packed weights, scales, activation tile) so that
// enough bytes are in flight to cover HBM latency, and a short one of expanded 16 KB operand tiles.
//
// Warps: 0 TMA producer, 1 MMA issuer, 2 tensor-memory alloc, 4-7 epilogue, 8-15 expansion.

template <int MMA_N, int LSTAGES, int OSTAGES>
struct DecodeW4A16Config {
    static constexpr int THREADS = 512;
    static constexpr int EXPAND_WARPS = 8;
    static constexpr uint32_t OP_BYTES = 128 * 128;          // expanded weight tile: 128 rows x 64 values x 2 bytes
    static constexpr uint32_t X_BYTES = MMA_N * 128;
    static constexpr uint32_t X_REGION = X_BYTES < 1024 ? 1024 : X_BYTES;
    static constexpr uint32_t PK_BYTES = 128 * 32;           // packed weights of one stage
    static constexpr uint32_t SF_BYTES = 512;                // one atom: 128 rows x 4 block scales
    static constexpr uint32_t TX_BYTES = PK_BYTES + SF_BYTES + X_BYTES;
    static constexpr uint32_t OP_OFF = 0;
    static constexpr uint32_t X_OFF = OSTAGES * OP_BYTES;
    static constexpr uint32_t PK_OFF = X_OFF + LSTAGES * X_REGION;
    static constexpr uint32_t SF_OFF = PK_OFF + LSTAGES * PK_BYTES;
    static constexpr uint32_t RING_BYTES = SF_OFF + LSTAGES * SF_BYTES;
    static constexpr uint32_t TMEM_COLS = 64;
    static constexpr uint32_t NUM_BARS = 2 * LSTAGES + 2 * OSTAGES + 1;
    static constexpr uint32_t BAR_BYTES = 8 * NUM_BARS + 16;
    static constexpr uint32_t SMEM_BYTES = RING_BYTES + BAR_BYTES + 1024;
    static constexpr int MAX_SPLIT = RING_BYTES / (MMA_N * 128 * 4) + 1 < 8 ? RING_BYTES / (MMA_N * 128 * 4) + 1 : 8;
    static_assert(MMA_N % 16 == 0 && MMA_N >= 16 && MMA_N <= 64, "activation rows per instruction");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
    static_assert(MMA_N * 128 * 4 <= RING_BYTES, "fp32 output staging must fit the rings");
};

// Expands one stage: thread t of 256 takes half a row (32 values = 16 packed bytes, two block
// scales).  packed: [128][32] bytes, even k in the low nibble; sf_atom: the tiled scale layout,
// row r at byte (r % 32) * 16 + (r / 32) * 4; dst: shared-memory address of the operand tile
// (1024-byte aligned), 16-byte unit j of row r at unit j ^ (r % 8).
//
// fp16: cvt.e2m1x2 -> f16x2, one packed multiply by the block scale.
// bf16: the fp16 bit pattern of an E2M1 value, shifted right by three with the sign put back,
// read as bf16 is the value times 2^-112 (the exponent field keeps its bits, the bias grows by
// 112; zero stays zero; the three mantissa bits shifted out are zero).  The block scale is
// therefore prepared as bf16(scale * 2^112) (at most 2^121, in range) and one packed bf16
// multiply gives value * scale exactly.
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
        uint32_t o[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t h2 = cvt_e2m1x2_to_f16x2((words[c] >> (8 * b)) & 0xFFu);
            if constexpr (BF16) o[b] = mul_bf16x2(((h2 >> 3) & 0x0FFF0FFFu) | (h2 & 0x80008000u), s);
            else o[b] = mul_f16x2(h2, s);
        }
        const uint32_t addr = drow + (static_cast<uint32_t>((half * 4 + c) ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
    }
}

template <bool BF16, int MMA_N, int LSTAGES, int OSTAGES>
__global__ void __launch_bounds__(512, 1)
decode_w4a16_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const DecodeStreamParams p) {
    using Cfg = DecodeW4A16Config<MMA_N, LSTAGES, OSTAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - raw);

    const uint32_t bar_base = base + Cfg::RING_BYTES;
    auto load_full = [&](int s) { return bar_base + 8u * s; };
    auto load_empty = [&](int s) { return bar_base + 8u * (LSTAGES + s); };
    auto op_ready = [&](int s) { return bar_base + 8u * (2 * LSTAGES + s); };
    auto op_empty = [&](int s) { return bar_base + 8u * (2 * LSTAGES + OSTAGES + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * LSTAGES + 2 * OSTAGES);
    const uint32_t slot_off = Cfg::RING_BYTES + 8u * Cfg::NUM_BARS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + slot_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + slot_off + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    [[maybe_unused]] const long long t_entry = BLZ_T_NOW();
    const int n_tile = blockIdx.x / p.split;
    const int split_idx = blockIdx.x % p.split;
    const int ks_begin = split_idx * p.stages_per_split;
    const int ks_end = min(p.k_stages_total, ks_begin + p.stages_per_split);

    if (threadIdx.x == 0) {
        for (int s = 0; s < LSTAGES; ++s) { mbar_init(load_full(s), 1); mbar_init(load_empty(s), 1); }
        for (int s = 0; s < OSTAGES; ++s) { mbar_init(op_ready(s), Cfg::EXPAND_WARPS); mbar_init(op_empty(s), 1); }
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
    griddep_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol_stream = l2_policy_evict_first();
            const uint64_t pol_keep = l2_policy_evict_last();
            auto load_weights = [&](int ks, int stage) {
                mbar_arrive_expect_tx(load_full(stage), Cfg::TX_BYTES);
                tma_load_2d_hint(base + Cfg::PK_OFF + stage * Cfg::PK_BYTES, &tm_w, ks * 32, n_tile * 128, load_full(stage), pol_stream);
                bulk_load_1d(base + Cfg::SF_OFF + stage * Cfg::SF_BYTES, p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + ks) * 512, Cfg::SF_BYTES, load_full(stage));
            };
            // packed weights and their scales of the first ring do not depend on earlier kernels
            const int n_pre = min(ks_end - ks_begin, LSTAGES);
            for (int i = 0; i < n_pre; ++i) load_weights(ks_begin + i, i);
            griddep_wait();
            int stage = 0; uint32_t phase = 0;
            for (int ks = ks_begin; ks < ks_end; ++ks) {
                if (ks - ks_begin >= LSTAGES) {
                    if (!mbar_wait(load_empty(stage), phase ^ 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; break;
                    }
                    load_weights(ks, stage);
                }
                tma_load_2d_hint(base + Cfg::X_OFF + stage * Cfg::X_REGION, &tm_x, ks * 128, 0, load_full(stage), pol_keep);
                if (++stage == LSTAGES) { stage = 0; phase ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int ls = 0, os = 0; uint32_t ophase = 0;
            bool ok = true;
            for (int ks = ks_begin; ks < ks_end; ++ks) {
                // "expanded" implies "landed": the expansion warps waited for the stage's loads
                if (!mbar_wait(op_ready(os), ophase, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                }
                tc_fence_after_sync();
                const uint32_t sw = base + Cfg::OP_OFF + os * Cfg::OP_BYTES;
                const uint32_t sx = base + Cfg::X_OFF + ls * Cfg::X_REGION;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t accumulate = (ks != ks_begin || k != 0) ? 1u : 0u;
                    umma_f16(tmem_base, make_desc_k_sw128(sw + k * 32), make_desc_k_sw128(sx + k * 32), p.idesc, accumulate);
                }
                tc_commit(op_empty(os));
                tc_commit(load_empty(ls));
                if (++ls == LSTAGES) ls = 0;
                if (++os == OSTAGES) { os = 0; ophase ^= 1u; }
            }
            if (ok) tc_commit(acc_full_bar);
        }
        __syncwarp();
    } else if (warp >= 8) {
        const int t = threadIdx.x - 256;
        int ls = 0, os = 0; uint32_t lphase = 0, ophase = 0;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
            if (!mbar_wait(load_full(ls), lphase, abort_flag) || !mbar_wait(op_empty(os), ophase ^ 1u, abort_flag)) {
                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; break;
            }
            expand_w4_stage<BF16>(gen_base + Cfg::PK_OFF + ls * Cfg::PK_BYTES, gen_base + Cfg::SF_OFF + ls * Cfg::SF_BYTES,
                            base + Cfg::OP_OFF + os * Cfg::OP_BYTES, t);
            fence_proxy_async_smem();        // the tensor core reads the tile through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(op_ready(os));
            if (++ls == LSTAGES) { ls = 0; lphase ^= 1u; }
            if (++os == OSTAGES) { os = 0; ophase ^= 1u; }
        }
    }

    decode_epilogue<MMA_N>(p, base, gen_base, tmem_base, acc_full_bar, abort_flag, n_tile, split_idx, warp, lane, t_entry);
    decode_teardown(tmem_base, Cfg::TMEM_COLS, abort_flag, warp);
}

}  // namespace blz
