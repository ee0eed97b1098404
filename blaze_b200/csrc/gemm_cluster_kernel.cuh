// gemm_cluster_kernel.cuh -- persistent tcgen05 GEMM over CTA groups of CG = 1 or 2 SMs.
//
//   C[M,N] = epilogue( alpha * sum_k A[M,K] * B[N,K]^T )        (both operands K-major)
//
// A group of CG CTAs (one thread-block cluster) owns output tiles of (128*CG) x BN.  With CG = 2
// the pair issues cta_group::2 instructions: each CTA stages its own 128 rows of A and its own
// half of the B tile, so per CTA a pipeline stage is a third smaller than for a 128 x BN tile and
// more stages fit; each CTA accumulates its 128 rows x BN in its own tensor memory.
// No multicast loads: every CTA fetches its own tiles.
//
// Warp roles in every CTA (NVFP4: 12 or 16 warps, otherwise 8):
//   warp 0      TMA producer: A tile, B tile (its share) and scale-factor atoms -> stage ring,
//               completion on the CTA's own full barrier
//   warp 1      MMA issuer (leader CTA only): waits for the stage's ready barrier, issues four
//               tcgen05.mma (32 bytes of K each), commits to the stage's empty barrier in every CTA
//               of the group and, after the last stage, to the accumulator-full barriers
//   warp 2      tensor-memory alloc/free; for kinds without scale factors also the relay that turns
//               "my tiles landed" into one arrive on the leader's ready barrier
//   warps 4-7   epilogue: tcgen05.ld the CTA's 128 accumulator rows, alpha / bias / SiLU / residual,
//               narrow, swizzled store to a staging buffer, TMA store (row-strided direct stores
//               when C is not 16-byte aligned)
//   warps 12-15 NVFP4 with one accumulator buffer only: a second set of epilogue warps; the two
//               sets drain alternate column chunks, which halves the time the tensor pipe waits
//   warps 8-11  NVFP4 only: move the stage's scale factors shared memory -> registers -> tensor
//               memory (tcgen05.st) into that stage's own columns, then arrive on the leader's ready
//               barrier.  Measured on B200: a tcgen05.cp costs ~70 cycles of the tensor pipe whatever
//               its size and does not overlap MMAs, tcgen05.st from other warps runs beside them.
//
// Counterpart of Blaze's gemm_fp8_kernel (src/kernels/gemm_fp8_sm100.cu:204-264) and
// gemm_fp4_blkscaled_persistent_kernel (src/kernels/gemm_fp4_blkscaled_sm100.cu:507-624).
#pragma once

#include "common.cuh"

#ifndef BLZ_NVF4_OVERLAP
#define BLZ_NVF4_OVERLAP 1
#endif

namespace blz {

struct ClusterGemmParams {
    int M, N;
    int m_tiles, n_tiles;    // tiles of (128*CG) x BN
    int group_m;             // tile rasterisation: bands of this many M tiles are walked N-first
    int k_stages;            // ceil(K bytes per row / 128)
    int split_k;             // K splits: split s of M tile m is scheduled as M tile s * m_tiles_real + m and writes its
    int k_per_split;         //   fp32 partial sums to that row block of a scratch matrix; stages per split
    int m_tiles_real;        // M tiles of the problem itself (m_tiles counts all splits)
    uint32_t idesc;
    uint32_t idesc2;         // 384-wide tiles only: the second instruction of a K step (N = 128)
    int sfb_row_blocks;      // 128-row blocks the tiled scale factors of B hold
    int expand_bf16;         // W4A16: the activations' (and so the expanded weights') format, 1 = bf16, 0 = fp16
    const uint8_t* sfa;      // tiled scale factors of A: [row blocks of 128][sf_katoms][512]
    const uint8_t* sfb;      // tiled scale factors of B
    int sf_katoms;
    int use_tma_store;       // C (and its pitch) 16-byte aligned: epilogue stores through the output maps
    int n_dst;               // output maps in use: 1, or one per GPU for the fused all-gather
    // The tail of the schedule.  When the tiles do not fill the last wave of CTA groups, the tiles of that
    // partial wave are cut along K into `tail_split` units each, so that every group has work until the end:
    // scheduled indices [0, tail_first) are whole tiles, index tail_first + u is split u % tail_split of tile
    // tail_first + u / tail_split (tail_first = 0: every tile is cut -- few tiles and a long K).  All units run
    // in the same, last wave on different CTA groups.  A unit's CTAs store raw fp32 partial sums to their block
    // of a scratch array, publish them (one release per epilogue warp on the tile's counter), wait -- bounded --
    // until the counter shows every unit of the tile, and then each finishes its own slice of the tile's
    // columns: the sum over the units in unit order (results do not depend on timing), epilogue, store to C.
    int tail_first;          // = total_units when nothing is split
    int tail_split, tail_kps;   // units per tail tile; K stages per unit
    int total_units;         // scheduled indices in all
    float4* tail_scratch;    // [unit][CTA of the group][BN / 4 column groups][128 rows] of four fp32 sums
    uint32_t* tail_flags;    // [tail tile][CTA of the group]: releases so far, over all launches of the plan
    uint32_t tail_target;    // the counter value that says "all units of this launch have published"
    int clc;                 // tiles come from the hardware's launch queue (cluster launch control) instead of a fixed stride
    EpilogueParams epi;
    int* status;
};

// Tile order.  Tiles running at the same time should share operand panels through L2: the M tiles
// are cut into bands of `group_m`; inside a band the tile index walks M fastest, then N, so one
// wave of CTA groups covers a roughly square block of group_m x (wave / group_m) tiles instead of
// a thin stripe that re-reads all of A for every few columns of B.
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int& m_tile, int& n_tile) {
    const int band_tiles = group_m * n_tiles;
    const int band = tile / band_tiles;
    const int first_m = band * group_m;
    const int rows = min(m_tiles - first_m, group_m);
    const int in_band = tile - band * band_tiles;
    m_tile = first_m + in_band % rows;
    n_tile = in_band / rows;
}

// K range of a scheduled tile and the problem's own M tile behind it (see split_k above).
template <typename P>
__device__ __forceinline__ void tile_k_range(const P& p, int m_ext, int& m_tile, int& ks0, int& ks1) {
    const int sidx = m_ext / p.m_tiles_real;
    m_tile = m_ext - sidx * p.m_tiles_real;
    ks0 = sidx * p.k_per_split;
    ks1 = min(p.k_stages, ks0 + p.k_per_split);
}

// A scheduled index is a whole tile or, in the split tail, one K range of a tile: `unit` >= 0 names its row
// block of the partial-sum scratch matrix.
template <typename P>
__device__ __forceinline__ void resolve_unit(const P& p, int index, int& tile, int& unit, int& ks0, int& ks1) {
    if (index < p.tail_first) { tile = index; unit = -1; return; }
    const int u = index - p.tail_first;
    const int t = u / p.tail_split;
    tile = p.tail_first + t;
    unit = u;
    ks0 = (u - t * p.tail_split) * p.tail_kps;
    ks1 = min(p.k_stages, ks0 + p.tail_kps);
}

// Epilogue of one K-split unit of the tail, for one epilogue warp (all 32 lanes call it): raw sums to the unit's
// scratch block, accumulator handed back, partial sums published, then -- once every unit of the tile has
// published -- this unit's slice of the tile's column groups summed over the units in unit order, finished and
// stored to C.  False: the bounded wait for the other units ran out.
template <int CG, int BN, int SETS, int CSIZE>
__device__ __forceinline__ bool tail_unit_epilogue(float4* scratch, uint32_t* flags, uint32_t target, int split, int unit, int cta_in_group,
                                                uint32_t t_row, int eset, int r_local, uint32_t acc_empty, uint32_t leader_rank,
                                                const volatile int* abort_flag, EpilogueParams epi, int row0, int col0, int M, int N, uint32_t warp_smem) {
    constexpr int GROUPS4 = BN / 4;
    const int lane = threadIdx.x & 31;
    const int t_tail = unit / split, s_unit = unit - t_tail * split;
    const int e_out = epi.out_type;
    const long long e_ldc = epi.ldc;
    uint8_t* const e_c = reinterpret_cast<uint8_t*>(epi.C);
    // lanes are rows, so a warp's store of one column group is 512 contiguous bytes
    float4* dst = scratch + (static_cast<size_t>(unit) * CSIZE + cta_in_group) * (GROUPS4 * 128) + r_local;
    [[maybe_unused]] const long long ts0 = BLZ_T_NOW();
    // two 32-column groups per step: the second tensor-memory load is in flight while the first one's stores issue
    constexpr int STEP = 32 * SETS;
#pragma unroll 1
    for (int c0 = eset * 32; c0 < BN; c0 += 2 * STEP) {
        uint32_t acc[32], acc_b[32];
        const bool second = c0 + STEP < BN;
        tmem_ld32(t_row + c0, acc);
        if (second) tmem_ld32(t_row + c0 + STEP, acc_b);
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 8; ++k)
            dst[(c0 / 4 + k) * 128] = make_float4(__uint_as_float(acc[4 * k]), __uint_as_float(acc[4 * k + 1]), __uint_as_float(acc[4 * k + 2]), __uint_as_float(acc[4 * k + 3]));
        if (second) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                dst[((c0 + STEP) / 4 + k) * 128] = make_float4(__uint_as_float(acc_b[4 * k]), __uint_as_float(acc_b[4 * k + 1]), __uint_as_float(acc_b[4 * k + 2]), __uint_as_float(acc_b[4 * k + 3]));
        }
    }
    // nothing follows a unit, but the barrier protocol stays whole
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) {
        if constexpr (CG == 1) mbar_arrive(acc_empty); else mbar_arrive_cluster(acc_empty, leader_rank);
    }
    uint32_t* flag = flags + t_tail * CSIZE + cta_in_group;
    [[maybe_unused]] const long long ts1 = BLZ_T_NOW();
    __threadfence();
    __syncwarp();
    if (lane == 0) red_release_gpu_add_u32(flag, 1u);
    [[maybe_unused]] const long long ts2 = BLZ_T_NOW();
    if (!flag_wait_warp(flag, target, abort_flag)) return false;
    [[maybe_unused]] const long long ts3 = BLZ_T_NOW();
    // This unit's slice: whole pairs of column groups (16 bytes of a 16-bit row), the last units may get none.
    const int per = (((GROUPS4 + split - 1) / split) + 1) & ~1;
    const int g_begin = min(GROUPS4, s_unit * per), g_end = min(GROUPS4, g_begin + per);
    const float4* src = scratch + (static_cast<size_t>(t_tail) * split * CSIZE + cta_in_group) * (GROUPS4 * 128) + r_local;
    constexpr size_t UNIT_STRIDE = static_cast<size_t>(CSIZE) * (GROUPS4 * 128);
    // Eight column groups (32 columns) at a time: eight independent loads per unit are in flight, and the warp's
    // 32 rows x 32 finished columns turn through its 4 KB of the staging memory so that the stores to C are whole
    // row segments (lanes are rows in the scratch layout).  Measured for a 128 x 128 slice: loads 4-5 k cycles,
    // arithmetic and staging 1 k, stores 3 k.
    constexpr int BATCH = 8;
    const int esize = e_out == OUT_F32 ? 4 : 2;
    const int units_row = esize == 4 ? 8 : 4;              // 16-byte units of one row of a batch
    const int rows_pass = 32 / units_row;
    const int warp_row0 = row0 + (r_local & ~31);
#pragma unroll 1
    for (int g0 = g_begin + eset * BATCH; g0 < g_end; g0 += BATCH * SETS) {
        float4 a[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; ++j) a[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 2
        for (int sp = 0; sp < split; ++sp) {
            float4 x[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) x[j] = (g0 + j < g_end) ? __ldcg(src + sp * UNIT_STRIDE + (g0 + j) * 128) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < BATCH; ++j) { a[j].x += x[j].x; a[j].y += x[j].y; a[j].z += x[j].z; a[j].w += x[j].w; }
        }
        // finished values (the whole-tile epilogue's arithmetic on 32 consecutive columns: uniform branches per
        // batch -- the same steps written per element compiled to predicated code that cost 200 cycles an element)
        // -> this lane's row of the warp's block, 16-byte unit u at slot u ^ (row % 8)
        const uint32_t srow = warp_smem + static_cast<uint32_t>(lane) * 128u;
        uint32_t bits[32];
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
            bits[4 * j] = __float_as_uint(a[j].x); bits[4 * j + 1] = __float_as_uint(a[j].y);
            bits[4 * j + 2] = __float_as_uint(a[j].z); bits[4 * j + 3] = __float_as_uint(a[j].w);
        }
        float v[32];
        epilogue_math32(epi, bits, v, row0 + r_local, col0 + 4 * g0, M, N);
        if (esize == 4) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(srow + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4)), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3]) : "memory");
        } else {
            uint32_t w[16];
            if (e_out == OUT_BF16) {
#pragma unroll
                for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) w[i] = pack2_out(OUT_F16, v[2 * i], v[2 * i + 1]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4)), "r"(w[4 * j]), "r"(w[4 * j + 1]), "r"(w[4 * j + 2]), "r"(w[4 * j + 3]) : "memory");
        }
        __syncwarp();
        // out again with lanes along the row: `units_row` lanes per row, `rows_pass` rows per pass
        const int u = lane % units_row;
        const int elems_unit = 16 / esize;
        const int n_u = col0 + 4 * g0 + u * elems_unit;             // first column of this lane's unit
        const bool unit_live = 4 * g0 + u * elems_unit < 4 * g_end;  // the batch may reach past the slice
        const bool vec = unit_live && n_u + elems_unit <= N && ((reinterpret_cast<uintptr_t>(e_c) | static_cast<uintptr_t>(e_ldc * esize) | static_cast<uintptr_t>(n_u * esize)) & 15u) == 0;
        uint8_t* dst_row = e_c + ((static_cast<long long>(warp_row0) + lane / units_row) * e_ldc + n_u) * esize;
        const long long dst_step = static_cast<long long>(rows_pass) * e_ldc * esize;
#pragma unroll 4
        for (int r = lane / units_row; r < 32; r += rows_pass, dst_row += dst_step) {
            if (!unit_live || warp_row0 + r >= M || n_u >= N) continue;
            uint32_t w[4];
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                         : "r"(warp_smem + static_cast<uint32_t>(r) * 128u + ((static_cast<uint32_t>(u) ^ (static_cast<uint32_t>(r) & 7u)) << 4)) : "memory");
            if (vec) {
                *reinterpret_cast<uint4*>(dst_row) = make_uint4(w[0], w[1], w[2], w[3]);
            } else if (esize == 4) {
                for (int k = 0; k < 4 && n_u + k < N; ++k) reinterpret_cast<uint32_t*>(dst_row)[k] = w[k];
            } else {
                for (int k = 0; k < 8 && n_u + k < N; ++k) reinterpret_cast<uint16_t*>(dst_row)[k] = static_cast<uint16_t>(w[k >> 1] >> (16 * (k & 1)));
            }
        }
        __syncwarp();
    }
    if (r_local == 0 && eset == 0) { BLZ_T_STORE(9, ts1 - ts0); BLZ_T_STORE(10, ts2 - ts1); BLZ_T_STORE(11, ts3 - ts2); BLZ_T_STORE(12, BLZ_T_NOW() - ts3); }
    return true;
}

// Where the epilogue stores a tile.  Normally one map (C).  For the fused GEMM + all-gather every
// GPU of the box passes one map per GPU: map d describes this rank's column block inside GPU d's
// full [M, N_total] output (its own buffer or a peer's, mapped through CUDA IPC), and each staged
// chunk is written once per destination with plain TMA stores -- the NVLink traffic overlaps the
// main loop tile by tile instead of following the GEMM as a separate collective.
constexpr int BLZ_MAX_DST = 8;
struct alignas(64) OutputMaps {
    CUtensorMap m[BLZ_MAX_DST];
};

template <int KIND, int CG, int BN, int STAGES, int ACC_BUFS, int SHARE = 1>
struct ClusterGemmConfig {
    // SHARE = 2: two CTA pairs (a cluster of four, tile 512 x BN) need the same B tile; each CTA
    // fetches only half of its share from L2 and forwards it to the matching CTA of the other
    // pair through distributed shared memory (and receives the other half the same way), which
    // cuts the B bytes every SM pulls from L2 in two.
    // BN = 384 (NVFP4 CTA pairs only): one tile is a 256-wide and a 128-wide instruction per K
    // step over the same A tile, which brings the bytes pulled from L2 per FLOP down by 16 %
    // against 256x256 (48 KB for 128 x 384 per CTA and stage instead of 38 KB for 128 x 256) --
    // the pair kernels are bound by L2 -> SM traffic.  The accumulator takes 384 tensor-memory
    // columns, so the scale factors get two slots that alternate, not one per stage.
    static constexpr bool WIDE = (BN > 256);
    static constexpr int CLUSTER = CG * SHARE;
    static constexpr bool HAS_SF = (KIND == MMA_NVF4);
    // With a single accumulator buffer the epilogue is on the critical path: two sets of four
    // epilogue warps (warps 4-7 and 12-15) then drain alternate column chunks.
    // W4A16: B arrives as packed NVFP4 (32 bytes per row and stage) plus one 512-byte scale atom;
    // warps 8-15 expand it into the 16-bit operand tile and report the stage ready.
    static constexpr bool HAS_EXPAND = (KIND == MMA_W4A16);
    static constexpr int EPI_SETS = (HAS_SF && ACC_BUFS == 1) ? 2 : 1;
    static constexpr int THREADS = HAS_SF ? (EPI_SETS == 2 ? 512 : 384) : (HAS_EXPAND ? 512 : 256);
    static constexpr uint32_t A_BYTES = 128 * 128;
    static constexpr uint32_t B_ROWS = BN / CG;                        // rows of the B tile staged by one CTA
    static constexpr uint32_t B_BYTES = B_ROWS * 128;
    static constexpr uint32_t B_LOAD_ROWS = B_ROWS / SHARE;            // rows this CTA itself fetches from L2
    static constexpr uint32_t B_LOAD_BYTES = B_LOAD_ROWS * 128;
    static constexpr uint32_t SF_BLOCK_BYTES = 4 * 512;                // one 128-row block, four K atoms
    static constexpr uint32_t SFB_BLOCKS = BN / 128;                   // every CTA needs the scales of all BN columns
    static constexpr uint32_t SFA_BYTES = HAS_SF ? SF_BLOCK_BYTES : 0;
    static constexpr uint32_t SFB_BYTES = HAS_SF ? SFB_BLOCKS * SF_BLOCK_BYTES : 0;
    static constexpr uint32_t PK_BYTES = HAS_EXPAND ? B_ROWS * 32 : 0;              // packed weights of one stage (64 K values per row)
    static constexpr uint32_t PK_SF_BYTES = HAS_EXPAND ? 1024 : 0;                  // one scale atom (512 bytes), padded to keep stages 1024-aligned
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES + PK_BYTES + PK_SF_BYTES;
    static constexpr uint32_t TX_BYTES = HAS_EXPAND ? A_BYTES + PK_BYTES + 512 : STAGE_BYTES;   // what TMA delivers per stage
    static constexpr uint32_t OUT_BUF_BYTES = 128 * 128;               // 128 rows x 128 bytes
    static constexpr uint32_t OUT_BYTES = 2 * OUT_BUF_BYTES;
    // NVFP4 pairs with 256-wide tiles: one 256-column accumulator plus a scale-factor slot per stage
    // fill tensor memory, which leaves the tensor pipe idle while the epilogue drains.  OVERLAP
    // keeps two accumulators that share 160 columns -- buffer 0 in columns [0, 256), buffer 1 in
    // [96, 352) -- and three scale-factor slots behind them.  Tiles alternate between the buffers;
    // the epilogue drains the shared columns first (buffer 0 from its top, buffer 1 from its
    // bottom) and hands the accumulator back as soon as they are in registers, so the next
    // tile's MMAs run beside the rest of the drain.
    static constexpr bool OVERLAP = BLZ_NVF4_OVERLAP && HAS_SF && !WIDE && CG == 2 && BN == 256 && ACC_BUFS == 1;
    static constexpr uint32_t ACC_OVL_OFF = 96;                         // first column of buffer 1
    static constexpr uint32_t OVL_COLS = OVERLAP ? BN - ACC_OVL_OFF : BN;  // columns of a tile the next tile's accumulator also uses
    static constexpr uint32_t ACC_COLS = OVERLAP ? ACC_OVL_OFF + BN : ACC_BUFS * BN;
    static constexpr uint32_t SF_COLS = HAS_SF ? 16 + 4 * (BN / 32) : 0;  // per stage: A 4 per atom, B BN/32 per atom
    static constexpr uint32_t SF_BASE = ACC_COLS;
    // Scale-factor slots in tensor memory.  One per stage when they fit; otherwise a shorter ring whose
    // slot s is rewritten once the MMAs that read it (SF_SLOTS stages earlier) have completed.  Two slots
    // leave one stage time (520 cycles) for "MMA done -> helper sees it -> tcgen05.st -> ready -> MMA
    // thread sees it", which is not enough; three leave two stage times.
    static constexpr int SF_SLOTS = OVERLAP ? 3 : WIDE ? 2 : STAGES;
    static constexpr uint32_t TMEM_NEED = ACC_COLS + SF_SLOTS * SF_COLS;
    static constexpr uint32_t TMEM_COLS = tmem_cols_pow2(TMEM_NEED);
    // Dynamic tile scheduling (cluster launch control): the grid holds one cluster per tile; a running cluster
    // that finishes a tile cancels a cluster that has not started yet and takes its tile.  One scheduler thread
    // (leader CTA, warp 3) talks to the hardware and hands tile indices to every role of every CTA of the
    // cluster through a ring of SCHED_SLOTS slots in shared memory.
    static constexpr int SCHED_SLOTS = 2;
    static constexpr bool CLC_OK = (SHARE == 1) && !HAS_EXPAND;               // kernels that can run with p.clc
    // roles that take tile indices, per CTA: producer, epilogue warps, scale-factor warps; plus the MMA thread once
    static constexpr uint32_t SCHED_CONSUMERS = CG * (1 + 4 * EPI_SETS + (HAS_SF ? 4 : 0)) + 1;
    static constexpr uint32_t NUM_BARS = (SHARE == 2 ? 5 : 3) * STAGES + 2 * ACC_BUFS + 2 * SCHED_SLOTS + 1;
    static constexpr uint32_t BAR_BYTES = 8 * NUM_BARS + 16 + 16 + 16;          // + launch-control answer (16-byte aligned) + tile slots
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BYTES + BAR_BYTES + 1024;
    static constexpr uint32_t READY_COUNT = HAS_SF ? 4 * CG : HAS_EXPAND ? 4 * CG : CG;      // arrivals that make a stage ready for the MMA
    // DIRECT: the MMA thread waits on ONE barrier per stage, the leader's full barrier.  The operand tiles of
    // every CTA of the group report their bytes there (CTA pairs: cp.async.bulk.tensor.cta_group::2 with the
    // leader's barrier), and so do the scale-factor warps once a stage's scale factors sit in tensor memory.
    // The scale factors land on a barrier of their own (the ready barrier's slot), so their way into tensor
    // memory runs while the much larger operand tiles are still in flight.  No relay hop, no second poll:
    // what is left between "tiles landed" and "MMA issued" is one barrier round trip.
    // The 512-thread NVFP4 kernels are launched with 128 registers per thread (the whole register file).
    // The single-thread roles and the scale-factor warps need far fewer, the epilogue warps want three
    // 32-column groups of the accumulator in flight: the budgets are re-cut per warpgroup at kernel start.
    static constexpr bool REG_SPLIT = HAS_SF && EPI_SETS == 2;
    static constexpr int REGS_ROLES = 48, REGS_SF = 72, REGS_EPI = 192;      // warps 0-3 / 8-11 / 4-7 and 12-15
    static_assert(!REG_SPLIT || (THREADS == 512 && 128 * (REGS_ROLES + REGS_SF + 2 * REGS_EPI) <= 512 * 128), "register budgets exceed the launch-time pool");
    static constexpr bool DIRECT = (SHARE == 1) && !HAS_EXPAND;
    static constexpr uint32_t FULL_COUNT = DIRECT ? 1 + (HAS_SF ? 4 * CG : 0) : 1;
    static constexpr uint32_t AB_TX_BYTES = CG * (A_BYTES + B_BYTES);                          // DIRECT: operand bytes of the whole group per stage
    static_assert(CG == 1 || CG == 2, "CTA group of 1 or 2");
    static_assert(SHARE == 1 || (SHARE == 2 && CG == 2), "B sharing needs CTA pairs");
    static_assert(!HAS_EXPAND || (SHARE == 1 && B_ROWS == 128), "W4A16: every CTA expands one 128-row block of weights per stage");
    static_assert(STAGE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned");
    static_assert(TMEM_NEED <= 512, "accumulators and scale factors exceed tensor memory");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
    static_assert(B_ROWS % 8 == 0 && BN % 128 == 0 && BN <= 384, "tile width");
    static_assert(!WIDE || (KIND == MMA_NVF4 && CG == 2 && SHARE == 1 && ACC_BUFS == 1 && STAGES % 2 == 0), "384-wide tiles: NVFP4 CTA pairs only");
};

// TAIL: the instance that can run K-split units of the tail (plans that asked for them); the plain instance
// carries none of that code -- in the NVFP4 pair kernel the extra epilogue path cost the whole-tile path its
// registers (11.6 k -> 14.5 k cycles per 256x256 tile at K = 4096).
template <int KIND, int CG, int BN, int STAGES, int ACC_BUFS, int SHARE = 1, bool TAIL = false>
__global__ void __launch_bounds__(ClusterGemmConfig<KIND, CG, BN, STAGES, ACC_BUFS, SHARE>::THREADS, 1)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ OutputMaps out, const ClusterGemmParams p) {
    using Cfg = ClusterGemmConfig<KIND, CG, BN, STAGES, ACC_BUFS, SHARE>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;      // the same offset in every CTA of the cluster
    uint8_t* gen_base = smem_raw + (base - raw);

    const uint32_t out_base = base + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bar_base = out_base + Cfg::OUT_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto ready_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (3 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (3 * STAGES + ACC_BUFS + b); };
    // B sharing only: "my own part of B landed" and "the other pair's CTA can take my part"
    auto bpart_bar = [&](int s) { return bar_base + 8u * (3 * STAGES + 2 * ACC_BUFS + s); };
    auto partner_ready_bar = [&](int s) { return bar_base + 8u * (4 * STAGES + 2 * ACC_BUFS + s); };
    constexpr uint32_t SCHED_BAR0 = (SHARE == 2 ? 5 : 3) * STAGES + 2 * ACC_BUFS;
    auto sched_full_bar = [&](int s) { return bar_base + 8u * (SCHED_BAR0 + s); };
    auto sched_empty_bar = [&](int s) { return bar_base + 8u * (SCHED_BAR0 + Cfg::SCHED_SLOTS + s); };
    const uint32_t clc_bar = bar_base + 8u * (SCHED_BAR0 + 2 * Cfg::SCHED_SLOTS);
    const uint32_t slot_off = STAGES * Cfg::STAGE_BYTES + Cfg::OUT_BYTES + 8u * Cfg::NUM_BARS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + slot_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + slot_off + 4);
    const uint32_t clc_response = (base + slot_off + 16u + 15u) & ~15u;          // 16 bytes, written by the hardware
    const uint32_t sched_tile0 = clc_response + 16u;                            // SCHED_SLOTS x int

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = (Cfg::CLUSTER == 1) ? 0u : cluster_cta_rank();
    const uint32_t pair = rank / CG;                 // which CTA group of the cluster (0 unless B is shared)
    const uint32_t prank = rank % CG;                // position inside the CTA group
    const bool leader = (prank == 0);
    const uint32_t leader_rank = rank - prank;       // cluster rank of this group's leader
    const uint32_t partner = rank ^ CG;              // B sharing: the CTA of the other pair that needs the same B rows
    const uint16_t commit_mask = static_cast<uint16_t>(0x3u << (pair * 2));

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), Cfg::FULL_COUNT);
            mbar_init(ready_bar(s), Cfg::DIRECT ? 1 : Cfg::READY_COUNT);   // DIRECT + scale factors: "this CTA's scale factors landed"
            mbar_init(empty_bar(s), 1);
            if constexpr (SHARE == 2) { mbar_init(bpart_bar(s), 1); mbar_init(partner_ready_bar(s), 1); }
        }
        for (int b = 0; b < ACC_BUFS; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), 4 * CG * Cfg::EPI_SETS); }
        for (int s = 0; s < Cfg::SCHED_SLOTS; ++s) { mbar_init(sched_full_bar(s), 1); mbar_init(sched_empty_bar(s), Cfg::SCHED_CONSUMERS); }
        mbar_init(clc_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if constexpr (Cfg::CLUSTER > 1) cluster_sync_all();   // every CTA of the cluster is resident before a pair allocates
    if (warp == 2) {
        if constexpr (CG == 2) { tmem_alloc_pair(base + slot_off, Cfg::TMEM_COLS); tmem_relinquish_pair(); }
        else { tmem_alloc(base + slot_off, Cfg::TMEM_COLS); tmem_relinquish(); }
    }
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        prefetch_tensormap(&out.m[0]);
    }
    tc_fence_before_sync();
    if constexpr (Cfg::CLUSTER > 1) cluster_sync_all(); else __syncthreads();   // barriers of every CTA are initialised
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = p.total_units;            // scheduled indices: whole tiles, then the K-split units of the tail
    const int group = blockIdx.x / Cfg::CLUSTER, num_groups = gridDim.x / Cfg::CLUSTER;   // a cluster walks tiles of (128*CG*SHARE) x BN
    const bool use_clc = Cfg::CLC_OK && p.clc != 0;

    // Where a role gets its tiles from.  Static: tile = group, group + num_groups, ...  Dynamic: the scheduler's
    // ring; every role of the cluster reads every slot (the tile index, -1 = no more) and then frees it with one
    // arrive on the leader's empty barrier -- warp-wide roles through lane 0 once all lanes have read.
    struct TileFeed {
        int tile, stride, total, n;
        bool dyn, warp_wide;
        uint32_t full0, empty0_leader, tile0;
        const volatile int* abort_flag;
        __device__ __forceinline__ int take() {
            if (!dyn) { const int t = tile; tile += stride; return t < total ? t : -1; }
            const int s = n % Cfg::SCHED_SLOTS;
            const uint32_t par = static_cast<uint32_t>(n / Cfg::SCHED_SLOTS) & 1u;
            ++n;
            if (!mbar_wait_acquire_cluster(full0 + 8u * s, par, abort_flag)) return -1;
            int t;
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(t) : "r"(tile0 + 4u * s) : "memory");
            if (warp_wide) __syncwarp();
            if (!warp_wide || (threadIdx.x & 31) == 0) mbar_arrive_cluster_addr(empty0_leader + 8u * s);
            return t;
        }
    };
    auto make_feed = [&](bool warp_wide) {
        TileFeed f;
        f.tile = group; f.stride = num_groups; f.total = total_tiles; f.n = 0; f.dyn = use_clc; f.warp_wide = warp_wide;
        f.full0 = sched_full_bar(0); f.tile0 = sched_tile0; f.abort_flag = abort_flag;
        f.empty0_leader = (Cfg::CLUSTER > 1) ? mapa_shared(sched_empty_bar(0), leader_rank) : sched_empty_bar(0);
        return f;
    };


    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (every CTA)
        if constexpr (Cfg::REG_SPLIT) warpgroup_regs_dec<Cfg::REGS_ROLES>();
        if (elect_one()) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            [[maybe_unused]] const uint32_t leader_full0 = (Cfg::CLUSTER > 1) ? mapa_shared(full_bar(0), leader_rank) : full_bar(0);
            BLZ_T_DECL(t_wait_empty);
            [[maybe_unused]] const long long t_begin = BLZ_T_NOW();
            TileFeed feed = make_feed(false);
            for (int tile = feed.take(); ok && tile >= 0; tile = feed.take()) {
                int m_tile, n_tile;
                int m_ext, ks0, ks1, unit, u0 = 0, u1 = 0;
                if constexpr (TAIL) resolve_unit(p, tile, tile, unit, u0, u1); else unit = -1;
                tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_ext, n_tile);
                tile_k_range(p, m_ext, m_tile, ks0, ks1);
                if (unit >= 0) { ks0 = u0; ks1 = u1; }
                const int a_row = ((m_tile * SHARE + static_cast<int>(pair)) * CG + static_cast<int>(prank)) * 128;
                const int b_row = n_tile * BN + static_cast<int>(prank) * static_cast<int>(Cfg::B_ROWS) + static_cast<int>(pair) * static_cast<int>(Cfg::B_LOAD_ROWS);
                for (int ks = ks0; ks < ks1; ++ks) {
                    [[maybe_unused]] const long long te = BLZ_T_NOW();
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; ok = false; break;
                    }
                    BLZ_T_ADD(t_wait_empty, te);
                    const uint32_t sa = base + stage * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    // where this stage's bytes report: DIRECT -> the leader's full barrier (operands) and my own
                    // scale-factor barrier; otherwise my own full barrier
                    [[maybe_unused]] const uint32_t ab_bar = (Cfg::DIRECT && CG == 2) ? leader_full0 + 8u * stage : full_bar(stage);
                    const uint32_t sf_tx_bar = Cfg::DIRECT ? ready_bar(stage) : full_bar(stage);
                    auto load_ab = [&](uint32_t dst, const CUtensorMap* m, int c0, int c1) {
                        if constexpr (Cfg::DIRECT && CG == 2) tma_load_2d_pair(dst, m, c0, c1, ab_bar);
                        else tma_load_2d(dst, m, c0, c1, full_bar(stage));
                    };
                    if constexpr (SHARE == 2) {
                        // everything but my own part of B completes on full_bar: A, scale factors and
                        // the part the partner forwards; my own part has its own barrier so that the
                        // forwarder can pass it on the moment it lands
                        mbar_arrive_expect_tx(full_bar(stage), Cfg::STAGE_BYTES - Cfg::B_LOAD_BYTES);
                        mbar_arrive_cluster(partner_ready_bar(stage), partner);    // my stage is free and armed: send
                    } else if constexpr (Cfg::DIRECT) {
                        if constexpr (Cfg::HAS_SF) mbar_arrive_expect_tx(sf_tx_bar, Cfg::SFA_BYTES + Cfg::SFB_BYTES);
                        if (leader) mbar_arrive_expect_tx(full_bar(stage), Cfg::AB_TX_BYTES);
                    } else {
                        mbar_arrive_expect_tx(full_bar(stage), Cfg::TX_BYTES);
                    }
                    if constexpr (Cfg::HAS_SF) {
                        // the small scale-factor copies go first: the helper warps need them before the MMA needs the tiles
                        const uint32_t ssfa = sb + Cfg::B_BYTES;
                        const uint32_t ssfb = ssfa + Cfg::SFA_BYTES;
                        const size_t katom = static_cast<size_t>(ks) * 4;
                        const size_t a_blk = (static_cast<size_t>(m_tile) * SHARE + pair) * CG + prank;
                        bulk_load_1d(ssfa, p.sfa + (a_blk * p.sf_katoms + katom) * 512, Cfg::SF_BLOCK_BYTES, sf_tx_bar);
#pragma unroll
                        for (int blk = 0; blk < static_cast<int>(Cfg::SFB_BLOCKS); ++blk) {
                            // a ragged last tile may reach past the last block: any valid block will do, those columns are never stored
                            const size_t rb = static_cast<size_t>(min(n_tile * static_cast<int>(Cfg::SFB_BLOCKS) + blk, p.sfb_row_blocks - 1));
                            bulk_load_1d(ssfb + blk * Cfg::SF_BLOCK_BYTES, p.sfb + (rb * p.sf_katoms + katom) * 512, Cfg::SF_BLOCK_BYTES, sf_tx_bar);
                        }
                    }
                    load_ab(sa, &tm_a, ks * 128, a_row);
                    if constexpr (SHARE == 2) {
                        // The partner's "ready" for this round also says that it has consumed what I
                        // forwarded last round, so my part of the stage may be overwritten now.
                        if (!mbar_wait(partner_ready_bar(stage), phase, abort_flag)) {
                            atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; ok = false; break;
                        }
                        mbar_arrive_expect_tx(bpart_bar(stage), Cfg::B_LOAD_BYTES);
                        tma_load_2d(sb + pair * Cfg::B_LOAD_BYTES, &tm_b, ks * 128, b_row, bpart_bar(stage));
                    } else if constexpr (Cfg::HAS_EXPAND) {
                        // packed weights of this CTA's 128 rows (32 bytes = 64 K values per row) and their scale atom
                        const uint32_t spk = sb + Cfg::B_BYTES;
                        tma_load_2d(spk, &tm_b, ks * 32, b_row, full_bar(stage));
                        const size_t rb = static_cast<size_t>(n_tile) * (BN / 128) + prank;
                        bulk_load_1d(spk + Cfg::PK_BYTES, p.sfb + (rb * p.sf_katoms + static_cast<size_t>(ks)) * 512, 512, full_bar(stage));
                    } else if constexpr (Cfg::WIDE) {
                        // this CTA's share of the 256-wide instruction (128 rows, two boxes of 64) and of the 128-wide one (64 rows)
                        const int n0 = n_tile * BN;
                        load_ab(sb, &tm_b, ks * 128, n0 + static_cast<int>(prank) * 128);
                        load_ab(sb + 8192, &tm_b, ks * 128, n0 + static_cast<int>(prank) * 128 + 64);
                        load_ab(sb + 16384, &tm_b, ks * 128, n0 + 256 + static_cast<int>(prank) * 64);
                    } else {
                        load_ab(sb, &tm_b, ks * 128, b_row);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            BLZ_T_STORE(0, t_wait_empty); BLZ_T_STORE(1, BLZ_T_NOW() - t_begin);
        }
        __syncwarp();
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer (leader CTA)
        if constexpr (Cfg::REG_SPLIT) warpgroup_regs_dec<Cfg::REGS_ROLES>();
        if (leader && elect_one()) {
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            [[maybe_unused]] uint32_t sslot = 0;   // scale-factor slot of the next stage (a ring of SF_SLOTS)
            [[maybe_unused]] int tr_n = 0;
            bool ok = true;
            BLZ_T_DECL(t_wait_ready); BLZ_T_DECL(t_wait_acc);
            [[maybe_unused]] const long long t_begin = BLZ_T_NOW();
            TileFeed feed = make_feed(false);
            for (int tile = feed.take(); ok && tile >= 0; tile = feed.take(), ++it) {
                const int buf = it % ACC_BUFS;
                const uint32_t use = static_cast<uint32_t>(it / ACC_BUFS);
                // The tile's first stage was loaded long ago (the producer runs ahead through the ring): its barrier
                // is looked at BEFORE the accumulator's, so that this poll's round trip (about 200 cycles even on a
                // completed phase) is spent while the epilogue still drains, not after it has handed the accumulator back.
                if (!mbar_wait(Cfg::DIRECT ? full_bar(stage) : ready_bar(stage), phase, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                }
                [[maybe_unused]] const long long ta = BLZ_T_NOW();
                if (!mbar_wait(acc_empty_bar(buf), (use & 1u) ^ 1u, abort_flag)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_ACC); *abort_flag = 1; ok = false; break;
                }
                BLZ_T_ADD(t_wait_acc, ta);
                BLZ_TRACE(1, it);
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (Cfg::OVERLAP ? static_cast<uint32_t>(it & 1) * Cfg::ACC_OVL_OFF : static_cast<uint32_t>(buf) * BN);
                int ks0, ks1;
                if (TAIL && tile >= p.tail_first) { int t_, u_; resolve_unit(p, tile, t_, u_, ks0, ks1); }     // a K-split unit of the tail
                else if (p.split_k == 1) { ks0 = 0; ks1 = p.k_stages; }      // no K split: nothing to look up (the divisions below would sit on the tile's critical path)
                else { int m_e, n_e, m_r; tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_e, n_e); tile_k_range(p, m_e, m_r, ks0, ks1); }
                for (int ks = ks0; ks < ks1; ++ks) {
                    [[maybe_unused]] const long long tr = BLZ_T_NOW();
                    if (ks != ks0 && !mbar_wait(Cfg::DIRECT ? full_bar(stage) : ready_bar(stage), phase, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                    }
                    BLZ_T_ADD(t_wait_ready, tr);
                    BLZ_TRACE(0, tr_n); ++tr_n;
                    tc_fence_after_sync();
                    const uint32_t sa = base + stage * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    const uint32_t sf_cols = tmem_base + Cfg::SF_BASE + (Cfg::SF_SLOTS == STAGES ? static_cast<uint32_t>(stage) : sslot) * Cfg::SF_COLS;
                    if (++sslot == static_cast<uint32_t>(Cfg::SF_SLOTS)) sslot = 0;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t ad = make_desc_k_sw128(sa + k * 32);
                        const uint64_t bd = make_desc_k_sw128(sb + k * 32);
                        const uint32_t accumulate = (ks != ks0 || k != 0) ? 1u : 0u;
                        if constexpr (Cfg::WIDE) {
                            // columns [0, 256) and [256, 384) of the tile; scale columns of one K atom: 8 + 4
                            umma_nvf4_pair(d_tmem, ad, bd, p.idesc, sf_cols + 4 * k, sf_cols + 16 + k * 12, accumulate);
                            umma_nvf4_pair(d_tmem + 256, ad, make_desc_k_sw128(sb + 16384 + k * 32), p.idesc2, sf_cols + 4 * k, sf_cols + 16 + k * 12 + 8, accumulate);
                        } else if constexpr (CG == 1) {
                            if constexpr (KIND == MMA_F16 || KIND == MMA_W4A16) umma_f16(d_tmem, ad, bd, p.idesc, accumulate);
                            else if constexpr (KIND == MMA_F8) umma_f8(d_tmem, ad, bd, p.idesc, accumulate);
                            else umma_nvf4(d_tmem, ad, bd, p.idesc, sf_cols + 4 * k, sf_cols + 16 + k * (BN / 32), accumulate);
                        } else {
                            if constexpr (KIND == MMA_F16 || KIND == MMA_W4A16) umma_f16_pair(d_tmem, ad, bd, p.idesc, accumulate);
                            else if constexpr (KIND == MMA_F8) umma_f8_pair(d_tmem, ad, bd, p.idesc, accumulate);
                            else umma_nvf4_pair(d_tmem, ad, bd, p.idesc, sf_cols + 4 * k, sf_cols + 16 + k * (BN / 32), accumulate);
                        }
                    }
                    if constexpr (CG == 1) tc_commit(empty_bar(stage)); else tc_commit_pair(empty_bar(stage), commit_mask);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) {
                    if constexpr (CG == 1) tc_commit(acc_full_bar(buf)); else tc_commit_pair(acc_full_bar(buf), commit_mask);
                }
            }
            BLZ_T_STORE(2, t_wait_ready); BLZ_T_STORE(3, t_wait_acc); BLZ_T_STORE(4, BLZ_T_NOW() - t_begin); BLZ_T_STORE(8, it);
        }
        __syncwarp();
    } else if (warp == 2) {
        // ----------------------------------- relay for kinds without scale factors (every CTA)
        if constexpr (Cfg::REG_SPLIT) warpgroup_regs_dec<Cfg::REGS_ROLES>();
        if constexpr (!Cfg::HAS_SF && !Cfg::HAS_EXPAND && !Cfg::DIRECT) {
            if (lane == 0) {
                int stage = 0; uint32_t phase = 0;
                bool ok = true;
                for (int tile = group; ok && tile < total_tiles; tile += num_groups) {
                    int ks0, ks1;
                    if (p.split_k == 1) { ks0 = 0; ks1 = p.k_stages; }      // no K split: nothing to look up (the divisions below would sit on the tile's critical path)
                else { int m_e, n_e, m_r; tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_e, n_e); tile_k_range(p, m_e, m_r, ks0, ks1); }
                    for (int ks = ks0; ks < ks1; ++ks) {
                        bool landed = mbar_wait(full_bar(stage), phase, abort_flag);
                        if constexpr (SHARE == 2) landed = landed && mbar_wait(bpart_bar(stage), phase, abort_flag);
                        if (!landed) {
                            atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                        }
                        if constexpr (CG == 1) mbar_arrive(ready_bar(stage)); else mbar_arrive_cluster(ready_bar(stage), leader_rank);
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            __syncwarp();
        }
    } else if (warp == 3) {
        // ------------------- B sharing: pass my part of every B stage on to the other pair's CTA
        if constexpr (Cfg::REG_SPLIT) warpgroup_regs_dec<Cfg::REGS_ROLES>();
        if constexpr (SHARE == 2) {
            if (elect_one()) {
                int stage = 0; uint32_t phase = 0;
                bool ok = true;
                for (int tile = group; ok && tile < total_tiles; tile += num_groups) {
                    int ks0, ks1;
                    if (p.split_k == 1) { ks0 = 0; ks1 = p.k_stages; }      // no K split: nothing to look up (the divisions below would sit on the tile's critical path)
                else { int m_e, n_e, m_r; tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_e, n_e); tile_k_range(p, m_e, m_r, ks0, ks1); }
                    for (int ks = ks0; ks < ks1; ++ks) {
                        if (!mbar_wait(bpart_bar(stage), phase, abort_flag)) {
                            atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; ok = false; break;
                        }
                        // The partner announced that its stage is free and armed before my producer
                        // even requested this part (it waited for partner_ready first).
                        const uint32_t part = base + stage * Cfg::STAGE_BYTES + Cfg::A_BYTES + pair * Cfg::B_LOAD_BYTES;
                        dsmem_copy(part, part, Cfg::B_LOAD_BYTES, full_bar(stage), partner);
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            __syncwarp();
        }
        if constexpr (Cfg::CLC_OK) {
            // ------------------------------------- tile scheduler (leader CTA, dynamic scheduling only)
            if (use_clc && leader && elect_one()) {
                int tile = group;                      // the tile this cluster was launched for
                bool ok = true;
#pragma unroll 1
                for (uint32_t n = 0; ok; ++n) {
                    const int s = static_cast<int>(n % Cfg::SCHED_SLOTS);
                    // the slot is free once every role of every CTA has read what it held
                    if (n >= static_cast<uint32_t>(Cfg::SCHED_SLOTS) &&
                        !mbar_wait(sched_empty_bar(s), ((n / Cfg::SCHED_SLOTS) - 1u) & 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; break;
                    }
#pragma unroll
                    for (uint32_t c = 0; c < static_cast<uint32_t>(CG); ++c) {
                        const uint32_t cta = leader_rank + c;
                        st_shared_cluster_u32(Cfg::CLUSTER > 1 ? mapa_shared(sched_tile0 + 4u * s, cta) : sched_tile0 + 4u * s, static_cast<uint32_t>(tile));
                        mbar_arrive_release_cluster_addr(Cfg::CLUSTER > 1 ? mapa_shared(sched_full_bar(s), cta) : sched_full_bar(s));
                    }
                    if (tile < 0) break;
                    // ask the launch queue for a cluster that has not started; its first CTA's x index names the tile
                    mbar_arrive_expect_tx(clc_bar, 16);
                    clc_try_cancel(clc_response, clc_bar);
                    if (!mbar_wait(clc_bar, n & 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_PRODUCER); *abort_flag = 1; break;
                    }
                    const int x = clc_query(clc_response);
                    tile = x < 0 ? -1 : x / Cfg::CLUSTER;
                }
            }
            __syncwarp();
        }
    } else if ((warp >= 4 && warp < 8) || (Cfg::EPI_SETS == 2 && warp >= 12)) {
        // ---------------------------------------------------------------- epilogue (every CTA)
        if constexpr (Cfg::REG_SPLIT) warpgroup_regs_inc<Cfg::REGS_EPI>();      // waits for what the other warpgroups hand back
        const int q = warp & 3;
        const int eset = warp >= 12 ? 1 : 0;                       // which set of four epilogue warps
        const int epi_tid = threadIdx.x - (eset ? 384 : 128);
        const uint32_t bar_id = 1 + eset;
        int it = 0;
        int obuf = 0;
        bool ok = true;
        BLZ_T_DECL(t_wait); BLZ_T_DECL(t_work);
        [[maybe_unused]] const long long t_begin = BLZ_T_NOW();
        TileFeed feed = make_feed(true);
        for (int tile = feed.take(); tile >= 0; tile = feed.take(), ++it) {
            int m_tile, n_tile, unit, u0_, u1_;
            if constexpr (TAIL) resolve_unit(p, tile, tile, unit, u0_, u1_); else unit = -1;
            tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_tile, n_tile);
            // a unit of the split tail stores raw fp32 partial sums to its row block of the scratch matrix
            const bool part = TAIL && unit >= 0;
            const EpilogueParams& epi = p.epi;
            const int out_esize = epi.out_type == OUT_F32 ? 4 : 2;
            const int chunk_cols = 128 / out_esize;                    // columns per 128-byte staging row
            const int buf = it % ACC_BUFS;
            const uint32_t use = static_cast<uint32_t>(it / ACC_BUFS);
            [[maybe_unused]] const long long tw = BLZ_T_NOW();
            if (ok && !mbar_wait(acc_full_bar(buf), use & 1u, abort_flag)) {
                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_EPILOGUE); *abort_flag = 1; ok = false;
            }
            BLZ_T_ADD(t_wait, tw);
            if (epi_tid == 0 && eset == 0) BLZ_TRACE(2, 8 * it);
            [[maybe_unused]] const long long tk = BLZ_T_NOW();
            // After a give-up the warps still walk the same named-barrier sequence (without touching
            // tensor memory or C) so that no epilogue warp is left waiting for another.
            tc_fence_after_sync();
            const int row0 = ((m_tile * SHARE + static_cast<int>(pair)) * CG + static_cast<int>(prank)) * 128;
            // where the staged chunks go: C (column n_tile * BN + c, row row0) or the unit's block of the scratch matrix
            const int st_col0 = n_tile * BN;
            const int st_row0 = row0;
            const int st_map0 = 0, st_maps = p.n_dst;
            const int r_local = q * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + (Cfg::OVERLAP ? static_cast<uint32_t>(it & 1) * Cfg::ACC_OVL_OFF : static_cast<uint32_t>(buf) * BN);
            if (part) {
              if constexpr (TAIL) {
                // ---- a K-split unit of the tail (always this group's last piece of work)
                // the staging memory (free once the earlier TMA stores have read it) becomes each warp's 4 KB transposition block
                if (epi_tid == 0) tma_store_wait_read<0>();
                named_barrier_sync(bar_id, 128);
                const uint32_t warp_smem = out_base + (Cfg::EPI_SETS == 2 ? eset : 0) * Cfg::OUT_BUF_BYTES + static_cast<uint32_t>(q) * 4096u;
                if (ok && !tail_unit_epilogue<CG, BN, Cfg::EPI_SETS, CG * SHARE>(p.tail_scratch, p.tail_flags, p.tail_target, p.tail_split, unit,
                                                                                static_cast<int>(pair) * CG + static_cast<int>(prank), t_row, eset, r_local,
                                                                                acc_empty_bar(buf), leader_rank, abort_flag, epi, row0, n_tile * BN, p.M, p.N, warp_smem)) {
                    atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_SPLITK); *abort_flag = 1; ok = false;
                }
              }
            } else if (p.use_tma_store) {
                if constexpr (Cfg::EPI_SETS == 2) {
                // (single accumulator barrier pair: the epilogue is on the tensor pipe's critical path until
                // it hands the accumulator back)
                // The two sets take alternate chunks of the drain order.  The accumulator reads run ahead of
                // the staging: the next chunk's columns are taken into registers as soon as the registers of
                // the current chunk's halves have been staged, and the accumulator goes back to the MMA role
                // right after this warp's last read of columns the next tile needs -- no wait for a staging
                // buffer or a TMA store sits between "accumulator full" and "accumulator free".
                // With overlapping accumulators those columns are the first OVL_COLS of the drain order:
                // buffer 0 (even tiles) drains from its top, buffer 1 from its bottom.
                const bool two = chunk_cols == 64;                         // 16-bit outputs: 64 columns per chunk, read as two halves of 32
                const int n_chunks = BN / chunk_cols;
                const bool down = Cfg::OVERLAP && (it & 1) == 0;
                auto chunk_col = [&](int j) { return down ? BN - (j + 1) * chunk_cols : j * chunk_cols; };
                const int hf = (two && down) ? 32 : 0;                     // the half of a chunk that comes first in drain order
                const int n_ov = (static_cast<int>(Cfg::OVL_COLS) + chunk_cols - 1) / chunk_cols;     // chunks that hold shared columns
                const int j_rel = ((n_ov - 1 - eset) / 2) * 2 + eset;      // this set's last such chunk
                // the shared columns end inside the first half of that chunk: release without waiting for the second
                const bool rel_first = two && static_cast<int>(Cfg::OVL_COLS) - j_rel * chunk_cols <= 32;
                uint32_t acc0[32], acc1[32];
                auto release = [&]() {
                    if (epi_tid == 0) BLZ_TRACE(3, 2 * it + eset);
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CG == 1) mbar_arrive(acc_empty_bar(buf)); else mbar_arrive_cluster(acc_empty_bar(buf), leader_rank);
                    }
                };
                const float alpha = epi.alpha;
                const bool plain16 = epi.mode == EPI_NONE && out_esize == 2;   // scale and narrow only: no temporaries, a handful of instructions per column pair
                const bool plain_bf16 = plain16 && epi.out_type == OUT_BF16;
                auto stage32 = [&](const uint32_t (&a)[32], uint32_t sbuf, int c, int h) {
                    // 128-byte swizzle: 16-byte unit j of row r lives at unit (j ^ (r % 8))
                    const uint32_t srow = sbuf + r_local * 128;
                    if (plain16) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t w[4];
                            if (plain_bf16) {
#pragma unroll
                                for (int t = 0; t < 4; ++t) w[t] = pack_bf16x2(__uint_as_float(a[8 * j + 2 * t]) * alpha, __uint_as_float(a[8 * j + 2 * t + 1]) * alpha);
                            } else {
#pragma unroll
                                for (int t = 0; t < 4; ++t) w[t] = pack2_out(OUT_F16, __uint_as_float(a[8 * j + 2 * t]) * alpha, __uint_as_float(a[8 * j + 2 * t + 1]) * alpha);
                            }
                            const uint32_t dst = srow + (((h / 8 + j) ^ (r_local & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                        }
                        return;
                    }
                    float v[32];
                    epilogue_math32(epi, a, v, row0 + r_local, n_tile * BN + c + h, p.M, p.N);
                    if (out_esize == 4) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t dst = srow + (((h / 4 + j) ^ (r_local & 7)) << 4);
                            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3]) : "memory");
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t w[4];
#pragma unroll
                            for (int t = 0; t < 4; ++t) w[t] = pack2_out(epi.out_type, v[8 * j + 2 * t], v[8 * j + 2 * t + 1]);
                            const uint32_t dst = srow + (((h / 8 + j) ^ (r_local & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                        }
                    }
                };
                // one staged chunk: wait for the set's staging buffer, stage both halves, hand the buffer to a store
                auto emit = [&](int c0, const uint32_t (&first)[32], const uint32_t (&second)[32], auto&& between) {
                    if (epi_tid == 0) tma_store_wait_read<0>();
                    named_barrier_sync(bar_id, 128);
                    const uint32_t sbuf = out_base + eset * Cfg::OUT_BUF_BYTES;
                    if (ok) {
                        stage32(first, sbuf, c0, hf);
                        stage32(second, sbuf, c0, hf ^ 32);
                        between();
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(bar_id, 128);
                    if (epi_tid == 0) {
                        if (ok) {
                            for (int d = 0; d < st_maps; ++d) tma_store_2d(&out.m[st_map0 + d], sbuf, (st_col0 + c0) * out_esize, st_row0);
                        }
                        tma_store_commit();
                    }
                };
                bool drained = false;
                if constexpr (Cfg::OVERLAP) {
                    if (two) {
                        // 16-bit output, four chunks of 64 columns; the next tile's accumulator shares the first 160
                        // columns of the drain order = chunks 0, 1 and the first half of chunk 2.  Set 1 takes chunks
                        // 1 and 3, set 0 chunks 0 and 2 -- and set 0 reads that first half of chunk 2 together with
                        // chunk 0 (a third group of 32 registers), so both sets release right after their first
                        // tcgen05.wait::ld: the tensor pipe waits for two loads, not for any arithmetic.
                        drained = true;
                        const int ca = chunk_col(eset), cb = chunk_col(eset + 2);
                        if (eset == 0) {
                            uint32_t acc2[32];
                            if (ok) {
                                tmem_ld32(t_row + ca + hf, acc0);
                                tmem_ld32(t_row + ca + (hf ^ 32), acc1);
                                tmem_ld32(t_row + cb + hf, acc2);
                                tmem_ld_wait();
                                if (epi_tid == 0) BLZ_TRACE(2, 8 * it + 2);
                                release();
                            }
                            emit(ca, acc0, acc1, [&]() { tmem_ld32(t_row + cb + (hf ^ 32), acc0); tmem_ld_wait(); });
                            emit(cb, acc2, acc0, [&]() {});
                        } else {
                            if (ok) {
                                tmem_ld32(t_row + ca + hf, acc0);
                                tmem_ld32(t_row + ca + (hf ^ 32), acc1);
                                tmem_ld_wait();
                                release();
                            }
                            uint32_t acc2[32];
                            emit(ca, acc0, acc1, [&]() { tmem_ld32(t_row + cb + hf, acc2); tmem_ld32(t_row + cb + (hf ^ 32), acc0); tmem_ld_wait(); });
                            emit(cb, acc2, acc0, [&]() {});
                        }
                    }
                }
                if (!drained && ok) {
                    const int c = chunk_col(eset);
                    tmem_ld32(t_row + c + hf, acc0);
                    if (two) tmem_ld32(t_row + c + (hf ^ 32), acc1);
                    tmem_ld_wait();
                    if (epi_tid == 0 && eset == 0) BLZ_TRACE(2, 8 * it + 2);
                    if (eset == j_rel) release();
                }
                for (int j = eset; !drained && j < n_chunks; j += Cfg::EPI_SETS) {
                    const int c0 = chunk_col(j);
                    const int jn = j + Cfg::EPI_SETS;
                    const bool more = ok && jn < n_chunks;
                    const int cn = more ? chunk_col(jn) : 0;
                    // each set owns one staging buffer: wait until its previous TMA store has finished reading it
                    if (epi_tid == 0) tma_store_wait_read<0>();
                    named_barrier_sync(bar_id, 128);
                    const uint32_t sbuf = out_base + eset * Cfg::OUT_BUF_BYTES;
                    if (epi_tid == 0 && eset == 0 && j == eset) BLZ_TRACE(2, 8 * it + 3);
                    if (ok) {
                        stage32(acc0, sbuf, c0, hf);
                        if (epi_tid == 0 && eset == 0 && j == eset) BLZ_TRACE(2, 8 * it + 4);
                        if (more) {
                            tmem_ld32(t_row + cn + hf, acc0);
                            if (jn == j_rel && rel_first) { tmem_ld_wait(); release(); }
                        }
                        if (two) {
                            stage32(acc1, sbuf, c0, hf ^ 32);
                            if (epi_tid == 0 && eset == 0 && j == eset) BLZ_TRACE(2, 8 * it + 5);
                            if (more) tmem_ld32(t_row + cn + (hf ^ 32), acc1);
                        }
                        if (more) {
                            tmem_ld_wait();
                            if (jn == j_rel && !rel_first) release();
                        }
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(bar_id, 128);
                    if (epi_tid == 0 && eset == 0 && j == eset) BLZ_TRACE(2, 8 * it + 6);
                    if (epi_tid == 0) {
                        if (ok) {
                            for (int d = 0; d < st_maps; ++d) tma_store_2d(&out.m[st_map0 + d], sbuf, (st_col0 + c0) * out_esize, st_row0);
                        }
                        tma_store_commit();
                    }
                    if (epi_tid == 0 && eset == 0 && j == eset) BLZ_TRACE(2, 8 * it + 7);
                }
                } else {
                // two accumulator buffers: the epilogue overlaps the next tile's MMAs; chunk by chunk
                for (int c0 = eset * chunk_cols; c0 < BN; c0 += chunk_cols * Cfg::EPI_SETS) {
                    // One set: the two staging buffers alternate, buffer `obuf` was handed to a TMA
                    // store two chunks ago.  Two sets: each set owns one buffer and waits for its own
                    // previous store.  Either way: wait until that store has finished reading it.
                    if (epi_tid == 0) { if constexpr (Cfg::EPI_SETS == 2) tma_store_wait_read<0>(); else tma_store_wait_read<1>(); }
                    named_barrier_sync(bar_id, 128);
                    const uint32_t sbuf = out_base + (Cfg::EPI_SETS == 2 ? eset : obuf) * Cfg::OUT_BUF_BYTES;
                    if (ok) {
                        for (int h = 0; h < chunk_cols; h += 32) {
                            uint32_t acc[32];
                            tmem_ld32(t_row + c0 + h, acc);
                            tmem_ld_wait();
                            if (c0 + chunk_cols * Cfg::EPI_SETS >= BN && h + 32 >= chunk_cols) {
                                // that was this warp's last read of the accumulator: hand it back to the
                                // MMA role now, the arithmetic and the stores of this chunk need it no more
                                tc_fence_before_sync();
                                __syncwarp();
                                if (lane == 0) {
                                    if constexpr (CG == 1) mbar_arrive(acc_empty_bar(buf)); else mbar_arrive_cluster(acc_empty_bar(buf), leader_rank);
                                }
                            }
                            const int col = n_tile * BN + c0 + h;
                            float v[32];
                            epilogue_math32(epi, acc, v, row0 + r_local, col, p.M, p.N);
                            // 128-byte swizzle: 16-byte unit j of row r lives at unit (j ^ (r % 8))
                            const uint32_t srow = sbuf + r_local * 128;
                            if (out_esize == 4) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const uint32_t dst = srow + (((h / 4 + j) ^ (r_local & 7)) << 4);
                                    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3]) : "memory");
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    uint32_t w[4];
#pragma unroll
                                    for (int t = 0; t < 4; ++t) w[t] = pack2_out(epi.out_type, v[8 * j + 2 * t], v[8 * j + 2 * t + 1]);
                                    const uint32_t dst = srow + (((h / 8 + j) ^ (r_local & 7)) << 4);
                                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                                }
                            }
                        }
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(bar_id, 128);
                    if (epi_tid == 0) {
                        if (ok) {
                            for (int d = 0; d < st_maps; ++d) tma_store_2d(&out.m[st_map0 + d], sbuf, (st_col0 + c0) * out_esize, st_row0);
                        }
                        tma_store_commit();
                    }
                    obuf ^= 1;
                }
                }
            } else if (ok) {
#pragma unroll 1
                for (int c0 = eset * 32; c0 < BN; c0 += 32 * Cfg::EPI_SETS) {
                    uint32_t acc[32];
                    tmem_ld32(t_row + c0, acc);
                    tmem_ld_wait();
                    epilogue_store32_dyn(epi, acc, row0 + r_local, n_tile * BN + c0, p.M, p.N);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (ok && !(p.use_tma_store || part) && lane == 0) {       // the other paths released the accumulator after their last read
                if constexpr (CG == 1) mbar_arrive(acc_empty_bar(buf)); else mbar_arrive_cluster(acc_empty_bar(buf), leader_rank);
            }
            BLZ_T_ADD(t_work, tk);
            if (epi_tid == 0 && eset == 0) BLZ_TRACE(2, 8 * it + 1);
        }
        if (epi_tid == 0 && eset == 0) { BLZ_T_STORE(5, t_wait); BLZ_T_STORE(6, t_work); BLZ_T_STORE(7, BLZ_T_NOW() - t_begin); }
        if (epi_tid == 0) tma_store_wait_all<0>();     // staging memory must outlive the last store's reads
    } else if (Cfg::HAS_EXPAND && warp >= 8) {
        // ------------- W4A16: packed weights + block scales -> 16-bit operand tile (warps 8-15)
        if constexpr (Cfg::HAS_EXPAND) {
            // Two groups of four warps take alternate stages (one stage's expansion is a chain of
            // barrier poll, loads, conversions, stores and a fence that outlasts the stage's MMAs);
            // inside a group every thread expands one weight row.
            const int eg = (warp - 8) >> 2;
            const int row = (threadIdx.x - 256) & 127;
            uint32_t n = 0;                                  // stages seen so far, over all tiles of this CTA
            bool ok = true;
            for (int tile = group; ok && tile < total_tiles; tile += num_groups) {
                int ks0, ks1;
                if (TAIL && tile >= p.tail_first) { int t_, u_; resolve_unit(p, tile, t_, u_, ks0, ks1); }     // a K-split unit of the tail
                else if (p.split_k == 1) { ks0 = 0; ks1 = p.k_stages; }      // no K split: nothing to look up (the divisions below would sit on the tile's critical path)
                else { int m_e, n_e, m_r; tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_e, n_e); tile_k_range(p, m_e, m_r, ks0, ks1); }
                for (int ks = ks0; ks < ks1; ++ks, ++n) {
                    if ((n & 1u) != static_cast<uint32_t>(eg)) continue;
                    const int stage = static_cast<int>(n % STAGES);
                    // landed = this stage's buffers were free (the producer waited for that) and TMA filled them
                    if (!mbar_wait_warp(full_bar(stage), (n / STAGES) & 1u, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                    }
                    const uint8_t* spk = gen_base + stage * Cfg::STAGE_BYTES + Cfg::A_BYTES + Cfg::B_BYTES;
                    const uint32_t sb = base + stage * Cfg::STAGE_BYTES + Cfg::A_BYTES;
                    if (p.expand_bf16) { expand_w4_stage<true>(spk, spk + Cfg::PK_BYTES, sb, 2 * row); expand_w4_stage<true>(spk, spk + Cfg::PK_BYTES, sb, 2 * row + 1); }
                    else { expand_w4_stage<false>(spk, spk + Cfg::PK_BYTES, sb, 2 * row); expand_w4_stage<false>(spk, spk + Cfg::PK_BYTES, sb, 2 * row + 1); }
                    fence_proxy_async_smem();        // the tensor core reads the tile through the async proxy
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CG == 1) mbar_arrive(ready_bar(stage)); else mbar_arrive_cluster(ready_bar(stage), leader_rank);
                    }
                }
            }
        }
    } else if (warp >= 8 && warp < 12) {
        // -------------------------------- NVFP4: scale factors smem -> registers -> tensor memory
        if constexpr (Cfg::REG_SPLIT) warpgroup_regs_dec<Cfg::REGS_SF>();
        if constexpr (Cfg::HAS_SF) {
            const int q = warp & 3;
            int stage = 0; uint32_t phase = 0;
            [[maybe_unused]] uint32_t g = 0;       // stages handled so far
            bool ok = true;
            TileFeed feed = make_feed(true);
            for (int tile = feed.take(); ok && tile >= 0; tile = feed.take()) {
                int ks0, ks1;
                if (TAIL && tile >= p.tail_first) { int t_, u_; resolve_unit(p, tile, t_, u_, ks0, ks1); }     // a K-split unit of the tail
                else if (p.split_k == 1) { ks0 = 0; ks1 = p.k_stages; }      // no K split: nothing to look up (the divisions below would sit on the tile's critical path)
                else { int m_e, n_e, m_r; tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, m_e, n_e); tile_k_range(p, m_e, m_r, ks0, ks1); }
                for (int ks = ks0; ks < ks1; ++ks) {
                    // DIRECT: only this CTA's scale factors have to have landed, the operand tiles may still be in flight
                    if (!mbar_wait(Cfg::DIRECT ? ready_bar(stage) : full_bar(stage), phase, abort_flag)) {
                        atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                    }
                    if constexpr (Cfg::SF_SLOTS < STAGES) {
                        // A ring of fewer slots than stages: slot g % SF_SLOTS was read by the MMAs of stage
                        // g - SF_SLOTS, whose completion the MMA role committed to that stage's empty barrier.
                        if (g >= static_cast<uint32_t>(Cfg::SF_SLOTS)) {
                            const uint32_t gp = g - Cfg::SF_SLOTS;
                            if (!mbar_wait(empty_bar(static_cast<int>(gp % STAGES)), (gp / STAGES) & 1u, abort_flag)) {
                                atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                            }
                            tc_fence_after_sync();
                        }
                    }
                    const uint8_t* ssfa = gen_base + stage * Cfg::STAGE_BYTES + Cfg::A_BYTES + Cfg::B_BYTES;
                    const uint8_t* ssfb = ssfa + Cfg::SFA_BYTES;
                    const uint32_t t_sf = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + Cfg::SF_BASE + (Cfg::SF_SLOTS == STAGES ? static_cast<uint32_t>(stage) : g % Cfg::SF_SLOTS) * Cfg::SF_COLS;
                    ++g;
                    {
                        uint32_t r[16];
#pragma unroll
                        for (int a = 0; a < 4; ++a) {
                            const uint4 v = *reinterpret_cast<const uint4*>(ssfa + a * 512 + lane * 16);
                            r[4 * a] = v.x; r[4 * a + 1] = v.y; r[4 * a + 2] = v.z; r[4 * a + 3] = v.w;
                        }
                        tmem_st16(t_sf, r);
                    }
                    if constexpr (BN == 384) {
                        // per K atom: 8 columns for the 256-wide instruction (blocks 0, 1), then 4 for the 128-wide one (block 2)
                        uint32_t r[48];
#pragma unroll
                        for (int a = 0; a < 4; ++a)
#pragma unroll
                            for (int blk = 0; blk < 3; ++blk) {
                                const uint4 v = *reinterpret_cast<const uint4*>(ssfb + blk * Cfg::SF_BLOCK_BYTES + a * 512 + lane * 16);
                                r[12 * a + 4 * blk] = v.x; r[12 * a + 4 * blk + 1] = v.y; r[12 * a + 4 * blk + 2] = v.z; r[12 * a + 4 * blk + 3] = v.w;
                            }
                        tmem_st32(t_sf + 16, *reinterpret_cast<const uint32_t(*)[32]>(&r[0]));
                        tmem_st16(t_sf + 48, *reinterpret_cast<const uint32_t(*)[16]>(&r[32]));
                    } else if constexpr (BN == 256) {
                        uint32_t r[32];
#pragma unroll
                        for (int a = 0; a < 4; ++a)
#pragma unroll
                            for (int blk = 0; blk < 2; ++blk) {
                                const uint4 v = *reinterpret_cast<const uint4*>(ssfb + blk * Cfg::SF_BLOCK_BYTES + a * 512 + lane * 16);
                                r[8 * a + 4 * blk] = v.x; r[8 * a + 4 * blk + 1] = v.y; r[8 * a + 4 * blk + 2] = v.z; r[8 * a + 4 * blk + 3] = v.w;
                            }
                        tmem_st32(t_sf + 16, r);
                    } else {
                        uint32_t r[16];
#pragma unroll
                        for (int a = 0; a < 4; ++a) {
                            const uint4 v = *reinterpret_cast<const uint4*>(ssfb + a * 512 + lane * 16);
                            r[4 * a] = v.x; r[4 * a + 1] = v.y; r[4 * a + 2] = v.z; r[4 * a + 3] = v.w;
                        }
                        tmem_st16(t_sf + 16, r);
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                    if constexpr (SHARE == 2) {
                        if (!mbar_wait(bpart_bar(stage), phase, abort_flag)) {
                            atomicCAS(p.status, 0, BLZ_DEV_TIMEOUT_MMA_FULL); *abort_flag = 1; ok = false; break;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        const uint32_t done_bar = Cfg::DIRECT ? full_bar(stage) : ready_bar(stage);
                        if constexpr (CG == 1) mbar_arrive(done_bar); else mbar_arrive_cluster(done_bar, leader_rank);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before_sync();
    if constexpr (Cfg::CLUSTER > 1) cluster_sync_all(); else __syncthreads();
    if (*abort_flag != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    if constexpr (Cfg::CLUSTER > 1) cluster_sync_all(); else __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        if constexpr (CG == 2) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS); else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace blz
