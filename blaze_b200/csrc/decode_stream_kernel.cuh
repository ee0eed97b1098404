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
    int k_stages_total;      // ceil(bytes of one weight row / 128)
    int stages_per_split;
    int split;               // = cluster size: 1, 2, 4 or 8
    uint32_t idesc;
    const uint8_t* sfw;      // tiled scale factors of the weights
    const uint8_t* sfx;      // tiled scale factors of the activations (row block 0)
    int sf_katoms;
    int l2_prefetch;         // weight stages beyond the first ring to pull into L2 before the wait for the predecessor grid
    int tiles_per_cta;       // W4A16 kernel for M <= 32 only: consecutive weight tiles per CTA (1 elsewhere)
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

// The 128 epilogue threads (threadIdx 128..255) write the staged fp32 sums stag[m][128] to C:
// alpha, bias / SiLU / residual, narrowing, 16-byte row stores.  Compact on purpose: it runs once.
__device__ __forceinline__ void decode_store_rows(const float* stag, int p_M, int p_N, int n_tile, float e_alpha, float e_alpha2, int e_mode, int e_out, int e_vec,
                                                  long long e_ldc, long long e_ldr, void* e_C, const void* e_bias, const void* e_res) {
                const int tid = threadIdx.x - 128;
                const int esize = e_out == OUT_F32 ? 4 : 2;
                // one item = 8 consecutive output columns of one row: 128 / 8 = 16 items per row; the fused
                // gate / up epilogue makes 64 outputs of the tile's 128 columns: 8 items per row
                const bool swiglu = e_mode == EPI_SWIGLU;
                const int ishift = swiglu ? 3 : 4;
                const int n_out = swiglu ? (p_N >> 1) : p_N;
    #pragma unroll 1
                for (int c = tid; c < (p_M << ishift); c += 128) {
                    const int m = c >> ishift, j = c & ((1 << ishift) - 1);
                    // columns of the staged tile this item reads, and the output column it writes
                    const int scol = swiglu ? ((j >> 1) * 32 + (j & 1) * 8) : j * 8;
                    const int col = swiglu ? (n_tile * 64 + j * 8) : (n_tile * 128 + j * 8);
                    if (col >= n_out) continue;
                    const float4 lo = *reinterpret_cast<const float4*>(stag + m * 128 + scol);
                    const float4 hi = *reinterpret_cast<const float4*>(stag + m * 128 + scol + 4);
                    float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    #pragma unroll
                    for (int t = 0; t < 8; ++t) v[t] *= e_alpha;
                    if (swiglu) {
                        // columns 32b .. 32b+15 of the GEMM are gate, 32b+16 .. 32b+31 up, of outputs 16b .. 16b+15
                        const float4 ulo = *reinterpret_cast<const float4*>(stag + m * 128 + scol + 16);
                        const float4 uhi = *reinterpret_cast<const float4*>(stag + m * 128 + scol + 20);
                        const float u[8] = {ulo.x, ulo.y, ulo.z, ulo.w, uhi.x, uhi.y, uhi.z, uhi.w};
    #pragma unroll
                        for (int t = 0; t < 8; ++t) v[t] = silu_f32(v[t]) * (u[t] * e_alpha2);
                    } else if (e_mode != EPI_NONE) {
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
                    const bool whole = e_vec && col + 8 <= n_out;
                    if (e_out == OUT_F32) {
                        if (whole) {
                            reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
                            reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
                        } else {
                            for (int t = 0; t < 8 && col + t < n_out; ++t) reinterpret_cast<float*>(dst)[t] = v[t];
                        }
                    } else {
                        uint32_t w[4];
    #pragma unroll
                        for (int t = 0; t < 4; ++t) w[t] = pack2_out(e_out, v[2 * t], v[2 * t + 1]);
                        if (whole) {
                            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                        } else {
                            for (int t = 0; t < 8 && col + t < n_out; ++t)
                                reinterpret_cast<uint16_t*>(dst)[t] = static_cast<uint16_t>(w[t >> 1] >> (16 * (t & 1)));
                        }
                    }
                }
}

// Shared by both kernels, called by every thread of the CTA once its main-loop role is done.
// Warps 4-7 take the fp32 sums out of tensor memory (columns [0, MMA_N), lane = weight row); with
// a K split every thread of every CTA of the cluster meets at two cluster barriers around the
// reduction through the leader's shared memory (at `base`, free once the main loops are over);
// the leader applies the epilogue and writes C.
template <int MMA_N, bool SLEEPY = false, int NACC = 1, int ACC_STRIDE = 64>
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
        epi_ok = SLEEPY ? mbar_wait_sleepy(acc_full_bar, 0u, abort_flag) : mbar_wait(acc_full_bar, 0u, abort_flag);
        BLZ_T_STORE_IF(threadIdx.x == 128, 5, clock64() - t_entry);
        if (!epi_ok) { atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_EPILOGUE); *abort_flag = 1; }
#pragma unroll
        for (int m = 0; m < MMA_N; ++m) acc[m] = 0.0f;
        if (epi_ok) {
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
            // NACC > 1: the kernel kept NACC independent partial accumulators ACC_STRIDE columns apart
            // (consecutive tcgen05.mma into one accumulator wait for each other); they are added
            // here in a fixed order.
#pragma unroll
            for (int a = 0; a < NACC; ++a) {
#pragma unroll
                for (int c = 0; c < MMA_N; c += 16) {
                    uint32_t r[16];
                    tmem_ld16(t_row + a * ACC_STRIDE + c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc[c + j] = a == 0 ? __uint_as_float(r[j]) : acc[c + j] + __uint_as_float(r[j]);
                }
            }
            tmem_ld_wait();
            tc_fence_before_sync();
        }
        BLZ_T_STORE_IF(threadIdx.x == 128, 1, clock64() - t_entry);
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
        BLZ_T_STORE_IF(threadIdx.x == 128, 2, clock64() - t_entry);
        griddep_wait();                      // bias / residual may come from the predecessor; C may be read by it
        named_barrier_sync(1, 128);          // all reads of the partial sums are done: the buffer can be reused
        float* stag = reinterpret_cast<float*>(gen_base);
#pragma unroll
        for (int m = 0; m < MMA_N; ++m) stag[m * 128 + n_local] = acc[m];
        named_barrier_sync(1, 128);
        BLZ_T_STORE_IF(threadIdx.x == 128, 6, clock64() - t_entry);
        if (epi_ok) {
            decode_store_rows(stag, p_M, p_N, n_tile, e_alpha, p.epi.alpha2, e_mode, e_out, e_vec, e_ldc, e_ldr, e_C, e_bias, e_res);
        }
    }

    BLZ_T_STORE_IF(threadIdx.x == 128, 7, clock64() - t_entry);
}

// The same for wide activation tiles (MMA_N = 128): the sums do not fit a thread's registers, so
// everything goes in chunks of 32 columns (= activation rows).  The NACC accumulators sit MMA_N
// columns apart.  The leader's staging buffer aliases partial-sum slot 0: every element of that
// slot is read (as a partial sum) and then overwritten (as the total) by the same thread.
template <int MMA_N, bool SLEEPY, int NACC>
__device__ __forceinline__ void decode_epilogue_wide(const DecodeStreamParams& p, uint32_t base, uint8_t* gen_base, uint32_t tmem_base,
                                                     uint32_t acc_full_bar, volatile int* abort_flag, int n_tile, int split_idx, int warp, int lane) {
    bool epi_ok = true;
    const bool is_epi = (warp >= 4 && warp < 8);
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    const float e_alpha = p.epi.alpha;
    const int e_mode = p.epi.mode, e_out = p.epi.out_type, e_vec = p.epi.vec_ok, p_M = p.M, p_N = p.N, p_split = p.split;
    const long long e_ldc = p.epi.ldc, e_ldr = p.epi.ldr;
    void* const e_C = p.epi.C;
    const void* const e_bias = p.epi.bias;
    const void* const e_res = p.epi.residual;
    if (is_epi) {
        epi_ok = SLEEPY ? mbar_wait_sleepy(acc_full_bar, 0u, abort_flag) : mbar_wait(acc_full_bar, 0u, abort_flag);
        if (!epi_ok) { atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_EPILOGUE); *abort_flag = 1; }
        tc_fence_after_sync();
    }
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    auto load_chunk = [&](int c, float (&v)[32]) {
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
            uint32_t r[32];
            tmem_ld32(t_row + a * MMA_N + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 32; ++t) v[t] = a == 0 ? __uint_as_float(r[t]) : v[t] + __uint_as_float(r[t]);
        }
    };
    if (p_split > 1) {
        cluster_sync_all();                 // every CTA of the tile is past its main loop: the leader's buffers are free
        if (is_epi && split_idx != 0 && epi_ok) {
#pragma unroll 1
            for (int c = 0; c < MMA_N && c < p_M; c += 32) {
                float v[32];
                load_chunk(c, v);
                const uint32_t dst = base + (static_cast<uint32_t>(split_idx - 1) * MMA_N * 128 + c * 128 + n_local) * 4;
#pragma unroll
                for (int t = 0; t < 32; ++t)
                    if (c + t < p_M) st_shared_cluster_f32(dst + t * 512, 0, v[t]);
            }
        }
        cluster_sync_all();                 // partial sums have landed in the leader
    }
    if (is_epi && split_idx == 0) {
        griddep_wait();                      // bias / residual may come from the predecessor; C may be read by it
        float* stag = reinterpret_cast<float*>(gen_base);
        if (epi_ok) {
#pragma unroll 1
            for (int c = 0; c < MMA_N && c < p_M; c += 32) {
                float v[32];
                load_chunk(c, v);
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    float sum = v[t];
                    for (int sp = 1; sp < p_split; ++sp) sum += stag[(sp - 1) * MMA_N * 128 + (c + t) * 128 + n_local];
                    stag[(c + t) * 128 + n_local] = sum;
                }
            }
        }
        tc_fence_before_sync();
        named_barrier_sync(1, 128);
        if (epi_ok) decode_store_rows(stag, p_M, p_N, n_tile, e_alpha, p.epi.alpha2, e_mode, e_out, e_vec, e_ldc, e_ldr, e_C, e_bias, e_res);
    }
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
    BLZ_T_STORE_IF(threadIdx.x == 0, 10, global_timer_ns());
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
    static constexpr uint32_t SF_BASE = MMA_N <= 64 ? 64 : 128;   // accumulator in columns [0, MMA_N)
    static constexpr uint32_t TMEM_COLS = HAS_SF ? tmem_cols_pow2(SF_BASE + STAGES * SF_COLS) : (MMA_N <= 64 ? 64 : 128);
    static constexpr uint32_t NUM_BARS = 3 * STAGES + 1;
    static constexpr uint32_t BAR_BYTES = 8 * NUM_BARS + 16;
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
    static constexpr int MAX_SPLIT = (STAGES * STAGE_BYTES) / (MMA_N * 128 * 4) + 1 < 8 ? (STAGES * STAGE_BYTES) / (MMA_N * 128 * 4) + 1 : 8;
    static_assert(MMA_N % 16 == 0 && MMA_N >= 16 && MMA_N <= 128, "activation rows per instruction");
    static_assert(!HAS_SF || SF_BASE + STAGES * SF_COLS <= TMEM_COLS, "scale-factor columns exceed the allocation");
    static_assert(MMA_N > 32 || SMEM_BYTES <= 115000, "two CTAs must fit one SM");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
    static_assert(TMEM_COLS <= 256 || SMEM_BYTES > 116 * 1024, "two CTAs on one SM would wait for each other's tensor memory");
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
    BLZ_T_STORE_IF(threadIdx.x == 0, 9, global_timer_ns());
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
    BLZ_T_STORE_IF(threadIdx.x == 0, 11, clock64() - t_entry);

    if (warp == 0) {
        if (elect_one()) {
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
            // ... and neither do the stages after them: while the predecessor grid drains (its epilogue
            // and completion leave HBM idle) they are pulled into L2, from where the ring refills faster
            const int pf_end = min(ks_end, ks_begin + n_pre + p.l2_prefetch);
            for (int ks = ks_begin + n_pre; ks < pf_end; ++ks) {
                tma_prefetch_l2_2d(&tm_w, ks * 128, n_tile * 128);
                if constexpr (Cfg::HAS_SF)
                    bulk_prefetch_l2(p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + static_cast<size_t>(ks) * 4) * 512, Cfg::SF_BYTES);
            }
            griddep_wait();
#ifdef BLZ_DECODE_LATE_DEPENDENTS
            griddep_launch_dependents();     // at most one successor prefetches while this grid runs
#endif
            BLZ_T_STORE(12, clock64() - t_entry); BLZ_T_STORE(14, global_timer_ns());
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
        if (elect_one()) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int ks = ks_begin; ks < ks_end; ++ks) {
                // without scale factors nothing stands between "landed" and "ready"
                if (!mbar_wait(Cfg::HAS_SF ? ready_bar(stage) : full_bar(stage), phase, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                }
                BLZ_T_STORE_IF(ks == ks_begin, 13, clock64() - t_entry);
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

    if constexpr (MMA_N > 64) decode_epilogue_wide<MMA_N, false, 1>(p, base, gen_base, tmem_base, acc_full_bar, abort_flag, n_tile, split_idx, warp, lane);
    else decode_epilogue<MMA_N>(p, base, gen_base, tmem_base, acc_full_bar, abort_flag, n_tile, split_idx, warp, lane, t_entry);
    decode_teardown(tmem_base, Cfg::TMEM_COLS, abort_flag, warp);
}

// ------------------------------------------------------------------------------------------------
// 16-bit activations x NVFP4 weights.
//
// The tensor core has no instruction that takes one 4-bit and one 16-bit operand, so the packed
// weights are expanded on the way, in the activations' 16-bit format (q * block scale: at most six
// significant bits, exact in fp16 and in bf16).  Both operands of a kind::f16 instruction must
// have the same format -- an fp16 A with a bf16 B is rejected by the hardware as an illegal
// instruction -- so bf16 activations need bf16 weights, which cost three more integer
// instructions per pair of values than fp16 (there is no E2M1 -> bf16 conversion).
//
// The expanded weights never touch shared memory: they are the instruction's A operand (128 weight
// rows = 128 tensor-memory lanes), and tcgen05.mma can read A from tensor memory.  Sixteen helper
// warps in four groups expand one sub-stage each (64 K values = 32 columns of packed 16-bit
// pairs) straight from the packed bytes in shared memory into registers and tcgen05.st them into
// a ring of operand slots next to the accumulator.  Measured on B200, the alternative -- writing a
// 16 KB swizzled operand tile per 64 K values to shared memory for the tensor core to read back --
// is bound by shared-memory bandwidth (a 128 x 16 x 16 MMA already spends 48 cycles reading its A
// tile from shared memory) and runs three times slower.  HBM only sees the 4.5 bits per weight.
//
// A load stage is what the NVFP4 kernel loads too: 128 weight rows x 128 packed bytes (256 K
// values; full 128-byte lines), their four 512-byte scale atoms, and the four activation tiles of
// those 256 K values.  It is consumed in four sub-stages of 64 K values, one group of four
// tcgen05.mma (K = 16 each) per sub-stage; expansion group g always takes sub-stage g.
//
// The tensor pipe is the bound.  Measured on B200: consecutive tcgen05.mma into the same
// accumulator wait for each other (~100 cycles apiece for a 128 x 16 x 16 instruction whose
// arithmetic is worth 8), so the four K = 16 slices of a sub-stage go to four independent
// accumulators that the epilogue adds; a tcgen05.commit costs ~45 cycles of the pipe, so the
// operand slots are handed back in groups of four (one commit per load stage, plus the one that
// frees the load stage) instead of one by one.
//
// Warps: 0 TMA producer, 1 MMA issuer, 2 tensor-memory alloc, 4-7 epilogue, 8-23 expansion
// (group = (warp - 8) / 4 = the sub-stage it takes; warp % 4 selects its 32 lanes).

template <int MMA_N, int LSTAGES>
struct DecodeW4A16Config {
    static constexpr int EXPAND_GROUPS = 4;                  // groups of four warps (one per 32 lanes)
    static constexpr int THREADS = 256 + 128 * EXPAND_GROUPS;
    static constexpr int SUBS = 4;                           // sub-stages (64 K values) per load stage
    // independent accumulators, one per K = 16 slice of a sub-stage, ACC_STRIDE columns apart; a CTA that
    // takes several weight tiles puts tile t at column offset t * MMA_N inside every stride
    static constexpr int NACC = 4;
    static constexpr uint32_t ACC_STRIDE = MMA_N <= 32 ? 32 : 64;
    static constexpr int MAX_TILES = ACC_STRIDE / MMA_N;
    static constexpr uint32_t OP_COL0 = ACC_STRIDE * NACC;
    static constexpr uint32_t OP_COLS = 32;                  // 64 K values x 16 bit per lane
    // operand slot groups in tensor memory, one per load stage in flight: whatever the accumulators leave
    static constexpr int OGROUPS = (512 - OP_COL0) / (SUBS * OP_COLS);
    static constexpr int OSLOTS = OGROUPS * SUBS;
    static constexpr uint32_t X_BYTES = MMA_N * 128;         // one activation tile (64 K values)
    static constexpr uint32_t X_REGION = X_BYTES < 1024 ? 1024 : X_BYTES;
    static constexpr uint32_t PK_BYTES = 128 * 128;          // packed weights of one load stage
    static constexpr uint32_t SF_BYTES = SUBS * 512;         // four atoms: 128 rows x 4 block scales each
    static constexpr uint32_t TX_BYTES = PK_BYTES + SF_BYTES + SUBS * X_BYTES;
    static constexpr uint32_t PK_OFF = 0;
    static constexpr uint32_t X_OFF = PK_OFF + LSTAGES * PK_BYTES;
    static constexpr uint32_t SF_OFF = X_OFF + LSTAGES * SUBS * X_REGION;
    static constexpr uint32_t RING_BYTES = SF_OFF + LSTAGES * SF_BYTES;
    static constexpr uint32_t TMEM_COLS = 512;               // the whole tensor memory: one CTA per SM (see SMEM_BYTES)
    static constexpr uint32_t NUM_BARS = 2 * LSTAGES + 2 * OGROUPS + 1;
    static constexpr uint32_t BAR_BYTES = 8 * NUM_BARS + 16;
    static constexpr uint32_t SMEM_BYTES = RING_BYTES + BAR_BYTES + 1024;
    static constexpr int MAX_SPLIT = RING_BYTES / (MMA_N * 128 * 4) + 1 < 8 ? RING_BYTES / (MMA_N * 128 * 4) + 1 : 8;
    static_assert(MMA_N % 16 == 0 && MMA_N >= 16 && MMA_N <= 64, "activation rows per instruction");
    static_assert(OP_COL0 + OSLOTS * OP_COLS <= TMEM_COLS, "operand slots exceed the allocation");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
    static_assert(MMA_N * 128 * 4 <= RING_BYTES, "fp32 output staging must fit the rings");
    static_assert(SMEM_BYTES > 116 * 1024, "two CTAs on one SM would wait for each other's tensor memory");
    static_assert(EXPAND_GROUPS == SUBS, "one expansion group per sub-stage");
};

// One thread expands the 64 K values of its weight row for one sub-stage into 32 registers of
// packed 16-bit pairs (lower k in the low half), the tensor-memory layout of a K-major A operand.
// packed_row: the row's 128 packed bytes of the load stage as a 128-byte-swizzled TMA load left
// them (16-byte unit u at unit u ^ (row % 8)), even k in the low nibble; sf4: the row's four
// block scales of this sub-stage (E4M3, lowest k first).
//
// fp16: cvt.e2m1x2 -> f16x2, one packed multiply by the block scale.
// bf16: the fp16 bit pattern of an E2M1 value, shifted right by three with the sign put back,
// read as bf16 is the value times 2^-112 (the exponent field keeps its bits, the bias grows by
// 112; zero stays zero; the three mantissa bits shifted out are zero).  The block scale is
// therefore prepared as bf16(scale * 2^112) (at most 2^121, in range) and one packed bf16
// multiply gives value * scale exactly.
template <bool BF16>
__device__ __forceinline__ void expand_w4_row(const uint8_t* packed_row, int row, int sub, uint32_t sf4, uint32_t (&r)[32]) {
    const uint4 w0 = *reinterpret_cast<const uint4*>(packed_row + (((sub * 2) ^ (row & 7)) << 4));
    const uint4 w1 = *reinterpret_cast<const uint4*>(packed_row + (((sub * 2 + 1) ^ (row & 7)) << 4));
    const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    const uint32_t s01 = cvt_e4m3x2_to_f16x2(static_cast<uint16_t>(sf4)), s23 = cvt_e4m3x2_to_f16x2(static_cast<uint16_t>(sf4 >> 16));
    uint32_t s[4];
    if constexpr (BF16) {
        const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&s01)), f23 = __half22float2(*reinterpret_cast<const __half2*>(&s23));
        const float big = __uint_as_float(0x77800000u);                    // 2^112
        s[0] = pack_bf16x2(f01.x * big, f01.x * big); s[1] = pack_bf16x2(f01.y * big, f01.y * big);
        s[2] = pack_bf16x2(f23.x * big, f23.x * big); s[3] = pack_bf16x2(f23.y * big, f23.y * big);
    } else {
        s[0] = __byte_perm(s01, 0, 0x1010); s[1] = __byte_perm(s01, 0, 0x3232);
        s[2] = __byte_perm(s23, 0, 0x1010); s[3] = __byte_perm(s23, 0, 0x3232);
    }
#pragma unroll
    for (int wd = 0; wd < 8; ++wd) {
        uint32_t h[4];
        cvt_e2m1x8_to_f16x2x4(words[wd], h);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if constexpr (BF16) r[4 * wd + b] = mul_bf16x2(((h[b] >> 3) & 0x0FFF0FFFu) | (h[b] & 0x80008000u), s[wd >> 1]);
            else r[4 * wd + b] = mul_f16x2(h[b], s[wd >> 1]);
        }
    }
}

template <bool BF16, int MMA_N, int LSTAGES>
__global__ void __launch_bounds__((DecodeW4A16Config<MMA_N, LSTAGES>::THREADS), 1)
decode_w4a16_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const DecodeStreamParams p) {
    using Cfg = DecodeW4A16Config<MMA_N, LSTAGES>;
    constexpr int SUBS = Cfg::SUBS, OSLOTS = Cfg::OSLOTS;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - raw);

    const uint32_t bar_base = base + Cfg::RING_BYTES;
    auto load_full = [&](int s) { return bar_base + 8u * s; };
    auto load_empty = [&](int s) { return bar_base + 8u * (LSTAGES + s); };
    auto og_ready = [&](int g) { return bar_base + 8u * (2 * LSTAGES + g); };
    auto og_empty = [&](int g) { return bar_base + 8u * (2 * LSTAGES + Cfg::OGROUPS + g); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * LSTAGES + 2 * Cfg::OGROUPS);
    const uint32_t slot_off = Cfg::RING_BYTES + 8u * Cfg::NUM_BARS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + slot_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + slot_off + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    [[maybe_unused]] const long long t_entry = BLZ_T_NOW();
    // A CTA takes p.tiles_per_cta consecutive weight tiles (every CTA of a cluster the same ones, each its
    // own K range): their load stages run through the rings as one sequence, each tile into accumulator
    // columns of its own; the epilogue, with its reduction over the cluster, then runs once per tile.
    const int n_tile = (blockIdx.x / p.split) * p.tiles_per_cta;
    const int n_own = min(p.tiles_per_cta, p.n_tiles - n_tile);
    const int split_idx = blockIdx.x % p.split;
    const int ks_begin = split_idx * p.stages_per_split;
    const int ks_end = min(p.k_stages_total, ks_begin + p.stages_per_split);
    const int n_load_tile = ks_end - ks_begin;
    const int n_load_all = n_load_tile * n_own;

    if (threadIdx.x == 0) {
        for (int s = 0; s < LSTAGES; ++s) { mbar_init(load_full(s), 1); mbar_init(load_empty(s), 1); }
        for (int g = 0; g < Cfg::OGROUPS; ++g) { mbar_init(og_ready(g), 4 * Cfg::EXPAND_GROUPS); mbar_init(og_empty(g), 1); }
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
        if (elect_one()) {
            const uint64_t pol_stream = l2_policy_evict_first();
            const uint64_t pol_keep = l2_policy_evict_last();
            auto load_weights = [&](int tile, int ks, int stage) {
                mbar_arrive_expect_tx(load_full(stage), Cfg::TX_BYTES);
                tma_load_2d_hint(base + Cfg::PK_OFF + stage * Cfg::PK_BYTES, &tm_w, ks * 128, tile * 128, load_full(stage), pol_stream);
                bulk_load_1d(base + Cfg::SF_OFF + stage * Cfg::SF_BYTES, p.sfw + (static_cast<size_t>(tile) * p.sf_katoms + static_cast<size_t>(ks) * SUBS) * 512,
                             Cfg::SF_BYTES, load_full(stage));
            };
            // packed weights and their scales of the first ring do not depend on earlier kernels
            const int n_pre = min(n_load_all, LSTAGES);
            {
                int tile = n_tile, ks = ks_begin;
                for (int i = 0; i < n_pre; ++i) {
                    load_weights(tile, ks, i);
                    if (++ks == ks_end) { ks = ks_begin; ++tile; }
                }
                // later stages of the first tile: into L2 while the predecessor grid drains
                if (n_pre < n_load_tile) {
                    const int pf_end = min(ks_end, ks_begin + n_pre + p.l2_prefetch);
                    for (int kp = ks_begin + n_pre; kp < pf_end; ++kp) {
                        tma_prefetch_l2_2d(&tm_w, kp * 128, n_tile * 128);
                        bulk_prefetch_l2(p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + static_cast<size_t>(kp) * SUBS) * 512, Cfg::SF_BYTES);
                    }
                }
            }
            griddep_wait();
            int stage = 0; uint32_t phase = 0;
            int tile = n_tile, ks = ks_begin;
            for (int li = 0; li < n_load_all; ++li) {
                if (li >= LSTAGES) {
                    if (!mbar_wait(load_empty(stage), phase ^ 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; break;
                    }
                    load_weights(tile, ks, stage);
                }
#pragma unroll
                for (int j = 0; j < SUBS; ++j)
                    tma_load_2d_hint(base + Cfg::X_OFF + (stage * SUBS + j) * Cfg::X_REGION, &tm_x, (ks * SUBS + j) * 128, 0, load_full(stage), pol_keep);
                if (++stage == LSTAGES) { stage = 0; phase ^= 1u; }
                if (++ks == ks_end) { ks = ks_begin; ++tile; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (elect_one()) {
            // This thread shares its scheduler with expansion warps, so its instruction count is on the
            // critical path: the loop is unrolled over one full period of both rings, which turns every
            // descriptor, tensor-memory address, barrier address and phase into "base + constant".
            constexpr int OGROUPS = Cfg::OGROUPS;
            constexpr int LPERIOD = (LSTAGES % (2 * OGROUPS) == 0) ? LSTAGES : (LSTAGES % 2 == 0 ? LSTAGES * OGROUPS : LSTAGES * 2 * OGROUPS);
            static_assert(LPERIOD % LSTAGES == 0 && LPERIOD % (2 * OGROUPS) == 0, "unroll period (load stages): rings and phases repeat");
            const uint64_t dx0 = make_desc_k_sw128(base + Cfg::X_OFF);
            const uint32_t a0 = tmem_base + Cfg::OP_COL0;
            const int n_load = n_load_all;
            bool ok = true;
            int li_tile = 0;                      // load stage within the current tile
            uint32_t acc0 = tmem_base;            // the current tile's accumulators
            BLZ_T_DECL(t_ready);
            for (int l0 = 0; ok && l0 < n_load; l0 += LPERIOD) {
#pragma unroll
                for (int ul = 0; ul < LPERIOD; ++ul) {
                    if (l0 + ul >= n_load) break;
                    const int ls = ul % LSTAGES, og = ul % OGROUPS;
                    const uint32_t ophase = static_cast<uint32_t>(ul / OGROUPS) & 1u;
                    // One wait per load stage: polling a barrier costs ~200 cycles even when its phase is
                    // long complete (measured), as much as issuing eight of these MMAs.
                    // "expanded" implies "landed": the expansion warps waited for the stage's loads.
                    [[maybe_unused]] const long long tr = BLZ_T_NOW();
                    if (!mbar_wait(og_ready(og), ophase, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                    }
                    BLZ_T_ADD(t_ready, tr);
                    tc_fence_after_sync();
#pragma unroll
                    for (int j = 0; j < SUBS; ++j) {
                        const int os = og * SUBS + j;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t accumulate = j != 0 ? 1u : (li_tile != 0 ? 1u : 0u);
                            // A: 16 K values = 8 columns of this slot; B: 32 bytes further into the activation tile
                            umma_f16_ts(acc0 + Cfg::ACC_STRIDE * k, a0 + os * Cfg::OP_COLS + k * 8, dx0 + (((ls * SUBS + j) * Cfg::X_REGION + k * 32) >> 4), p.idesc, accumulate);
                        }
                    }
                    if (!ok) break;
                    tc_commit(og_empty(og));        // the four operand slots of this load stage
                    tc_commit(load_empty(ls));      // its packed bytes were expanded before the MMAs, its activation tiles are read by them
                    if (++li_tile == n_load_tile) { li_tile = 0; acc0 += MMA_N; }     // next tile: next accumulator columns
                }
            }
            if (ok) tc_commit(acc_full_bar);
            BLZ_T_STORE(8, t_ready); BLZ_T_STORE(9, BLZ_T_NOW() - t_entry);
        }
        __syncwarp();
    } else if (warp >= 8) {
        const int j = (warp - 8) >> 2, q = warp & 3;               // group = the sub-stage it takes; which 32 tensor-memory lanes
        const int row = q * 32 + lane;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::OP_COL0;
        const int n_load = n_load_all;
        BLZ_T_DECL(t_load); BLZ_T_DECL(t_slot); BLZ_T_DECL(t_expand); BLZ_T_DECL(t_sync);
        for (int li = 0; li < n_load; ++li) {
            const int ls = li % LSTAGES, og = li % Cfg::OGROUPS, os = og * SUBS + j;
            const uint32_t lphase = static_cast<uint32_t>(li / LSTAGES) & 1u, ophase = static_cast<uint32_t>(li / Cfg::OGROUPS) & 1u;
            [[maybe_unused]] const long long t0 = BLZ_T_NOW();
            if (!mbar_wait_warp(load_full(ls), lphase, abort_flag)) {
                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; break;
            }
            BLZ_T_ADD(t_load, t0);
            [[maybe_unused]] const long long t1 = BLZ_T_NOW();
            uint32_t r[32];
            const uint32_t sf4 = *reinterpret_cast<const uint32_t*>(gen_base + Cfg::SF_OFF + ls * Cfg::SF_BYTES + j * 512 + lane * 16 + q * 4);
            expand_w4_row<BF16>(gen_base + Cfg::PK_OFF + ls * Cfg::PK_BYTES + row * 128, row, j, sf4, r);
            BLZ_T_ADD(t_expand, t1);
            [[maybe_unused]] const long long t2 = BLZ_T_NOW();
            // the slot group is free once the MMAs of the load stage that used it last have completed
            if (!mbar_wait_warp(og_empty(og), ophase ^ 1u, abort_flag)) {
                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; break;
            }
            tc_fence_after_sync();
            BLZ_T_ADD(t_slot, t2);
            [[maybe_unused]] const long long t3 = BLZ_T_NOW();
            tmem_st32(t_lane + os * Cfg::OP_COLS, r);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(og_ready(og));
            BLZ_T_ADD(t_sync, t3);
        }
        BLZ_T_STORE_IF(lane == 0 && q == 0 && j == 0, 0, t_load); BLZ_T_STORE_IF(lane == 0 && q == 0 && j == 0, 3, t_slot);
        BLZ_T_STORE_IF(lane == 0 && q == 0 && j == 0, 4, t_expand); BLZ_T_STORE_IF(lane == 0 && q == 0 && j == 0, 11, t_sync);
    }

    // the epilogue warps sleep between polls: the expansion warps need every issue slot
    for (int t = 0; t < n_own; ++t)
        decode_epilogue<MMA_N, true, Cfg::NACC, Cfg::ACC_STRIDE>(p, base, gen_base, tmem_base + t * MMA_N, acc_full_bar, abort_flag, n_tile + t, split_idx, warp, lane, t_entry);
    decode_teardown(tmem_base, Cfg::TMEM_COLS, abort_flag, warp);
}

// ------------------------------------------------------------------------------------------------
// The same kernel for 64 < M <= 128: one activation tile of 128 rows (the instruction's N).  The
// activation tiles are now the bigger part of the traffic into shared memory (16 KB per 64 K values,
// from L2), so they get a ring of their own, two sub-stages per slot, behind their own barriers;
// the packed weights keep their load stages.  Two accumulators of 128 columns (even / odd K = 16
// slice), eight operand slots: all 512 tensor-memory columns.

template <int WSTAGES, int XSLOTS>
struct DecodeW4A16WideConfig {
    static constexpr int MMA_N = 128;
    static constexpr int EXPAND_GROUPS = 4;
    static constexpr int THREADS = 256 + 128 * EXPAND_GROUPS;
    static constexpr int SUBS = 4;
    static constexpr int OGROUPS = 2;
    static constexpr int NACC = 2;
    static constexpr uint32_t X_TILE = MMA_N * 128;          // one activation tile (64 K values)
    static constexpr uint32_t X_SLOT = 2 * X_TILE;           // two sub-stages per slot
    static constexpr uint32_t PK_BYTES = 128 * 128;
    static constexpr uint32_t SF_BYTES = SUBS * 512;
    static constexpr uint32_t W_TX = PK_BYTES + SF_BYTES;
    static constexpr uint32_t PK_OFF = 0;
    static constexpr uint32_t X_OFF = PK_OFF + WSTAGES * PK_BYTES;
    static constexpr uint32_t SF_OFF = X_OFF + XSLOTS * X_SLOT;
    static constexpr uint32_t RING_BYTES = SF_OFF + WSTAGES * SF_BYTES;
    static constexpr uint32_t OP_COL0 = NACC * MMA_N;
    static constexpr uint32_t OP_COLS = 32;
    static constexpr uint32_t TMEM_COLS = 512;
    static constexpr uint32_t NUM_BARS = 2 * WSTAGES + 2 * XSLOTS + 2 * OGROUPS + 1;
    static constexpr uint32_t BAR_BYTES = 8 * NUM_BARS + 16;
    static constexpr uint32_t SMEM_BYTES = RING_BYTES + BAR_BYTES + 1024;
    // partial sums of the other splits: (split - 1) slots of MMA_N x 128 fp32 (slot 0 doubles as the staging buffer)
    static constexpr int MAX_SPLIT = RING_BYTES / (MMA_N * 128 * 4) + 1 < 8 ? RING_BYTES / (MMA_N * 128 * 4) + 1 : 8;
    static_assert(OP_COL0 + OGROUPS * SUBS * OP_COLS <= TMEM_COLS, "operand slots exceed tensor memory");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
    static_assert(SMEM_BYTES > 116 * 1024, "two CTAs on one SM would wait for each other's tensor memory");
    static_assert(MMA_N * 128 * 4 <= RING_BYTES, "fp32 output staging must fit the rings");
};

template <bool BF16, int WSTAGES, int XSLOTS>
__global__ void __launch_bounds__((DecodeW4A16WideConfig<WSTAGES, XSLOTS>::THREADS), 1)
decode_w4a16_wide_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const DecodeStreamParams p) {
    using Cfg = DecodeW4A16WideConfig<WSTAGES, XSLOTS>;
    constexpr int SUBS = Cfg::SUBS, OGROUPS = Cfg::OGROUPS, MMA_N = Cfg::MMA_N;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - raw);

    const uint32_t bar_base = base + Cfg::RING_BYTES;
    auto w_full = [&](int s) { return bar_base + 8u * s; };
    auto w_empty = [&](int s) { return bar_base + 8u * (WSTAGES + s); };
    auto x_full = [&](int s) { return bar_base + 8u * (2 * WSTAGES + s); };
    auto x_empty = [&](int s) { return bar_base + 8u * (2 * WSTAGES + XSLOTS + s); };
    auto og_ready = [&](int g) { return bar_base + 8u * (2 * WSTAGES + 2 * XSLOTS + g); };
    auto og_empty = [&](int g) { return bar_base + 8u * (2 * WSTAGES + 2 * XSLOTS + OGROUPS + g); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * WSTAGES + 2 * XSLOTS + 2 * OGROUPS);
    const uint32_t slot_off = Cfg::RING_BYTES + 8u * Cfg::NUM_BARS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + slot_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + slot_off + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tile = blockIdx.x / p.split;
    const int split_idx = blockIdx.x % p.split;
    const int ks_begin = split_idx * p.stages_per_split;
    const int ks_end = min(p.k_stages_total, ks_begin + p.stages_per_split);
    const int n_load = ks_end - ks_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < WSTAGES; ++s) { mbar_init(w_full(s), 1); mbar_init(w_empty(s), 1); }
        for (int s = 0; s < XSLOTS; ++s) { mbar_init(x_full(s), 1); mbar_init(x_empty(s), 1); }
        for (int g = 0; g < OGROUPS; ++g) { mbar_init(og_ready(g), 4 * Cfg::EXPAND_GROUPS); mbar_init(og_empty(g), 1); }
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
        if (elect_one()) {
            const uint64_t pol_stream = l2_policy_evict_first();
            const uint64_t pol_keep = l2_policy_evict_last();
            auto load_weights = [&](int ks, int stage) {
                mbar_arrive_expect_tx(w_full(stage), Cfg::W_TX);
                tma_load_2d_hint(base + Cfg::PK_OFF + stage * Cfg::PK_BYTES, &tm_w, ks * 128, n_tile * 128, w_full(stage), pol_stream);
                bulk_load_1d(base + Cfg::SF_OFF + stage * Cfg::SF_BYTES, p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + static_cast<size_t>(ks) * SUBS) * 512,
                             Cfg::SF_BYTES, w_full(stage));
            };
            const int n_pre = min(n_load, WSTAGES);
            for (int i = 0; i < n_pre; ++i) load_weights(ks_begin + i, i);
            // later stages: into L2 while the predecessor grid drains
            const int pf_end = min(ks_begin + n_load, ks_begin + n_pre + p.l2_prefetch);
            for (int ks = ks_begin + n_pre; ks < pf_end; ++ks) {
                tma_prefetch_l2_2d(&tm_w, ks * 128, n_tile * 128);
                bulk_prefetch_l2(p.sfw + (static_cast<size_t>(n_tile) * p.sf_katoms + static_cast<size_t>(ks) * SUBS) * 512, Cfg::SF_BYTES);
            }
            griddep_wait();
            bool ok = true;
            int xi = 0;
            for (int li = 0; ok && li < n_load; ++li) {
                const int ws = li % WSTAGES, ks = ks_begin + li;
                if (li >= WSTAGES) {
                    if (!mbar_wait(w_empty(ws), (static_cast<uint32_t>(li / WSTAGES) & 1u) ^ 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; break;
                    }
                    load_weights(ks, ws);
                }
                for (int h = 0; h < 2; ++h, ++xi) {
                    const int xs = xi % XSLOTS;
                    if (xi >= XSLOTS && !mbar_wait(x_empty(xs), (static_cast<uint32_t>(xi / XSLOTS) & 1u) ^ 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; ok = false; break;
                    }
                    mbar_arrive_expect_tx(x_full(xs), Cfg::X_SLOT);
                    tma_load_2d_hint(base + Cfg::X_OFF + xs * Cfg::X_SLOT, &tm_x, (ks * SUBS + 2 * h) * 128, 0, x_full(xs), pol_keep);
                    tma_load_2d_hint(base + Cfg::X_OFF + xs * Cfg::X_SLOT + Cfg::X_TILE, &tm_x, (ks * SUBS + 2 * h + 1) * 128, 0, x_full(xs), pol_keep);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (elect_one()) {
            const uint64_t dx0 = make_desc_k_sw128(base + Cfg::X_OFF);
            const uint32_t a0 = tmem_base + Cfg::OP_COL0;
            bool ok = true;
            int xi = 0;
            for (int li = 0; ok && li < n_load; ++li) {
                const int ws = li % WSTAGES, og = li % OGROUPS;
                // "expanded" implies "landed": the expansion warps waited for the stage's weight loads
                if (!mbar_wait(og_ready(og), static_cast<uint32_t>(li / OGROUPS) & 1u, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                }
                for (int h = 0; h < 2; ++h, ++xi) {
                    const int xs = xi % XSLOTS;
                    if (!mbar_wait(x_full(xs), static_cast<uint32_t>(xi / XSLOTS) & 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const int os = og * SUBS + 2 * h + jj;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            // even and odd K = 16 slices go to separate accumulators
                            const uint32_t accumulate = (li | h | jj | (k >> 1)) != 0 ? 1u : 0u;
                            umma_f16_ts(tmem_base + (k & 1) * MMA_N, a0 + os * Cfg::OP_COLS + k * 8,
                                        dx0 + ((xs * Cfg::X_SLOT + jj * Cfg::X_TILE + k * 32) >> 4), p.idesc, accumulate);
                        }
                    }
                    tc_commit(x_empty(xs));
                }
                if (!ok) break;
                tc_commit(og_empty(og));
                tc_commit(w_empty(ws));
            }
            if (ok) tc_commit(acc_full_bar);
        }
        __syncwarp();
    } else if (warp >= 8) {
        const int j = (warp - 8) >> 2, q = warp & 3;
        const int row = q * 32 + lane;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::OP_COL0;
        for (int li = 0; li < n_load; ++li) {
            const int ws = li % WSTAGES, og = li % OGROUPS, os = og * SUBS + j;
            if (!mbar_wait_warp(w_full(ws), static_cast<uint32_t>(li / WSTAGES) & 1u, abort_flag)) {
                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; break;
            }
            uint32_t r[32];
            const uint32_t sf4 = *reinterpret_cast<const uint32_t*>(gen_base + Cfg::SF_OFF + ws * Cfg::SF_BYTES + j * 512 + lane * 16 + q * 4);
            expand_w4_row<BF16>(gen_base + Cfg::PK_OFF + ws * Cfg::PK_BYTES + row * 128, row, j, sf4, r);
            if (!mbar_wait_warp(og_empty(og), (static_cast<uint32_t>(li / OGROUPS) & 1u) ^ 1u, abort_flag)) {
                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; break;
            }
            tc_fence_after_sync();
            tmem_st32(t_lane + os * Cfg::OP_COLS, r);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(og_ready(og));
        }
    }

    decode_epilogue_wide<MMA_N, true, Cfg::NACC>(p, base, gen_base, tmem_base, acc_full_bar, abort_flag, n_tile, split_idx, warp, lane);
    decode_teardown(tmem_base, Cfg::TMEM_COLS, abort_flag, warp);
}

}  // namespace blz
