/*
 * blaze_b200.h -- C ABI of the B200 (sm_100a) GEMM library.
 *
 * Plain C: pointers, sizes, enums.  Every data pointer is a DEVICE pointer owned by the caller
 * unless stated otherwise; `stream` arguments are cudaStream_t handles passed as void*.
 * Every function returns a blz_status; nothing here calls exit() or prints.
 *
 * The entry points replace, one for one, the host API Blaze declares under include/gemm/
 * (citations are paths inside the Blaze project):
 *
 *   blz_gemm_plan_create   <- create_fp8_gemm_plan            include/gemm/fp8_gemm_sm100.cuh:84
 *                             create_fp4_gemm_plan            include/gemm/fp4_gemm_sm100.cuh:114
 *                             create_fp4_blkscaled_gemm_plan  include/gemm/fp4_blkscaled_gemm_sm100.cuh:155
 *                             create_fp4_blkscaled_persistent_gemm_plan                      ...:198
 *                             create_mixed_gemm_plan          include/gemm/mixed_gemm_sm100.cuh:123
 *   blz_gemm_execute       <- execute_fp8_gemm :95, execute_fp4_gemm :126,
 *                             execute_fp4_blkscaled_gemm :163, execute_fp4_blkscaled_persistent_gemm :206,
 *                             execute_mixed_gemm :136
 *   blz_gemm_plan_destroy  <- destroy_*_plan (same headers)
 *   blz_gemm_launch        <- launch_gemm_fp8 :63, launch_gemm_fp4 :93, launch_gemm_fp4_blkscaled :138,
 *                             launch_gemm_fp4_blkscaled_persistent :180, launch_gemm_mixed :76
 *   blz_tile_scales        <- interleave_scales_kernel / interleave_scales_transposed_kernel
 *                             src/kernels/gemm_fp4_blkscaled_sm100.cu:59-104
 *
 * The C++ functions of namespace blaze with Blaze's own signatures are thin shims over this ABI
 * (include/gemm/ *.cuh in this repository).
 */
#ifndef BLAZE_B200_H
#define BLAZE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum blz_status {
    BLZ_OK = 0,
    BLZ_ERR_INVALID_ARGUMENT = 1, /* null pointer, non-positive size, misaligned pointer or pitch */
    BLZ_ERR_UNSUPPORTED = 2,      /* a combination this build has no kernel for */
    BLZ_ERR_CUDA = 3,             /* a CUDA runtime / driver call failed; see blz_last_cuda_error */
    BLZ_ERR_DEVICE_TIMEOUT = 4,   /* a kernel gave up on a bounded wait; its output is invalid */
    BLZ_ERR_NO_DEVICE = 5,        /* no sm_100 device is current */
    BLZ_ERR_TOO_LARGE = 6,        /* exceeds a stated maximum */
    BLZ_ERR_OUT_OF_MEMORY = 7
} blz_status;

/* What the two operands are.  A is always [M, K] row-major. */
typedef enum blz_gemm_kind {
    BLZ_GEMM_F16 = 0,       /* fp16 x fp16 */
    BLZ_GEMM_BF16 = 1,      /* bf16 x bf16 */
    BLZ_GEMM_FP8 = 2,       /* E4M3 x E4M3, one fp32 scale per tensor */
    BLZ_GEMM_NVFP4 = 3,     /* E2M1 x E2M1, E4M3 scale per 16 values along K, fp32 scale per tensor */
    BLZ_GEMM_W4A16_F16 = 4, /* fp16 activations x NVFP4 weights */
    BLZ_GEMM_W4A16_BF16 = 5 /* bf16 activations x NVFP4 weights */
} blz_gemm_kind;

typedef enum blz_dtype { BLZ_F16 = 0, BLZ_BF16 = 1, BLZ_F32 = 2 } blz_dtype;

/* Order: scale -> bias -> SiLU / residual -> narrow (Blaze: src/kernels/gemm_mixed_sm100.cu:202-229). */
typedef enum blz_epilogue {
    BLZ_EPI_NONE = 0,
    BLZ_EPI_BIAS = 1,
    BLZ_EPI_SILU = 2,
    BLZ_EPI_BIAS_SILU = 3,
    BLZ_EPI_RESIDUAL_ADD = 4,
    BLZ_EPI_SWIGLU = 5 /* fused gate + up projection (Blaze: launch_fused_gate_up,
                          include/gemm/mixed_gemm_sm100.cuh:87-109, a stub there).  B holds N = 2 * N_out
                          weight rows, gate and up rows interleaved in groups of 16 (rows 32b..32b+15:
                          gate rows 16b..16b+15; rows 32b+16..32b+31: up rows 16b..16b+15; see
                          blz_interleave_gate_up); N a multiple of 32.  C is [M, N/2] (ldc 0 = N/2):
                          C[m, j] = silu(a_scale*b_scale*gate[m, j]) * (a_scale*b_scale2*up[m, j]).
                          One kernel, every variant; no K split of the tiled kernel, not with
                          blz_gemm_execute_gather. */
} blz_epilogue;

typedef enum blz_b_layout {
    BLZ_B_KMAJOR = 0, /* B stored [N, K] row-major (K contiguous): used as is */
    BLZ_B_NMAJOR = 1  /* B stored [K, N] row-major as Blaze's headers describe it; the plan keeps a
                         K-major copy.  For 4-bit data two N-neighbours share a byte. */
} blz_b_layout;

typedef enum blz_sf_layout {
    BLZ_SF_ROWMAJOR = 0, /* A: [M, K/16]; B: [N, K/16] (K-major B) or [K/16, N] (N-major B) */
    BLZ_SF_TILED = 1     /* [ceil(rows/128)][katoms][512 bytes], see blz_tile_scales */
} blz_sf_layout;

typedef enum blz_variant {
    BLZ_VARIANT_AUTO = 0,
    BLZ_VARIANT_TILE_128x128 = 1, /* one CTA per 128x128 tile, two accumulator buffers */
    BLZ_VARIANT_PAIR_256x256 = 2, /* CTA pairs (cta_group::2), one 256x256 tile per pair */
    BLZ_VARIANT_DECODE = 3,       /* skinny M: weights as the 128-row operand, split along K.  AUTO picks it
                                     for M <= 64 (W4A16: M <= 128, expanding the packed weights in the
                                     kernel); on request also M <= 128 for FP8 and 16-bit, not NVFP4 */
    BLZ_VARIANT_QUAD_512x256 = 4, /* two CTA pairs per 512x256 tile; the pairs pass each other their
                                     halves of the B tile through distributed shared memory */
    BLZ_VARIANT_PAIR_256x384 = 5, /* NVFP4 only: CTA pairs, 256x384 tiles (a 256-wide and a 128-wide
                                     instruction per K step), fewer L2 bytes per FLOP */
    BLZ_VARIANT_PAIR_256x128 = 6  /* CTA pairs, 256x128 tiles: twice as many tiles as 256x256 for problems whose
                                     256x256 tiles fill the last wave of CTA pairs badly */
} blz_variant;

typedef enum blz_gemm_flags {
    BLZ_FLAG_CLC_SCHEDULER = 1, /* tiled variants: dynamic tile scheduling through cluster launch control
                                  (clusterlaunchcontrol.try_cancel) -- the grid holds one cluster per tile and
                                  running clusters take over the tiles of clusters that have not started --
                                  instead of the static persistent schedule.  What Blaze sketches in
                                  include/gemm/tmem_utils.cuh:251-305 and never wires (its persistent kernel
                                  claims tiles with atomicAdd, src/kernels/gemm_fp4_blkscaled_sm100.cu:555-563).
                                  Ignored by the 512x256 variant and by in-kernel W4A16 expansion. */
    BLZ_FLAG_TAIL_SPLIT = 4,    /* tiled variants: when the last wave of tiles is at most half full (or the whole problem has
                                  at most half as many tiles as the device has CTA groups), cut those tiles along K into
                                  units that keep every CTA group busy.  Inside the same launch the units of a tile
                                  exchange fp32 partial sums through plan-owned scratch memory and each finishes a slice
                                  of the tile, summing in unit order (run-to-run identical; not bit-identical to the
                                  whole-tile schedule).  The units of a tile wait for one another (bounded: a wait that
                                  runs out sets the plan's status), so the plan must be able to have its whole grid
                                  resident -- do not run it beside kernels that hold SMs for long.  Off by default:
                                  measured on B200 a unit's exchange costs about what 32 K stages of a 256x256 tile cost,
                                  so it pays only when k_stages * (1 - 1/units) is well above that (f16 512 x 12288 x 4096:
                                  59.0 -> 55.1 us; FP8 4096^3: 56.0 -> 58.3 us).  Ignored with several outputs
                                  (blz_gemm_execute_gather), the 512x256 and 256x384 variants, in-kernel W4A16 expansion,
                                  the fused gate / up epilogue and BLZ_FLAG_CLC_SCHEDULER. */
    BLZ_FLAG_STATIC_WEIGHTS = 2 /* W4A16, M > 128: the caller promises that the packed weights and their scales
                                  do not change while the plan lives (or calls blz_gemm_plan_refresh_weights
                                  after changing them).  The plan then expands them ONCE, at creation, into a
                                  plan-owned 16-bit copy (N*K*2 bytes) and every execute is one launch of the
                                  dense 16-bit kernel -- instead of expanding inside the kernel (M <= 2048) or
                                  re-expanding all weights on every execute (M > 2048).  Blaze's own mixed plan
                                  has the same contract: its create call converts operands once
                                  (src/kernels/gemm_mixed_sm100.cu:412-470). */
} blz_gemm_flags;

typedef struct blz_gemm_desc {
    int32_t kind;         /* blz_gemm_kind */
    int32_t out_dtype;    /* blz_dtype of C, bias and residual (bias is fp32 when C is fp32) */
    int32_t epilogue;     /* blz_epilogue */
    int32_t variant;      /* blz_variant, 0 = choose */
    int32_t M, N, K;      /* in elements */
    int32_t b_layout;     /* blz_b_layout */
    int32_t a_sf_layout;  /* blz_sf_layout (NVFP4 A only) */
    int32_t b_sf_layout;  /* blz_sf_layout (NVFP4 B / W4A16 weights) */
    const void* A;        /* [M, K] values, or packed E2M1 [M, K/2] (even K index in the low nibble) */
    const void* A_sf;     /* E4M3 block scales of A, or null */
    const void* B;        /* see b_layout */
    const void* B_sf;     /* E4M3 block scales of B, or null */
    float a_scale;        /* dequantisation multiplier of A: x ~ code * a_scale (1 for fp16/bf16) */
    float b_scale;        /* same for B.  alpha = a_scale * b_scale is applied to the accumulator */
    const void* bias;     /* [N] or null */
    const void* residual; /* [M, ldc] or null */
    int64_t ldc;          /* row pitch of C and residual in elements; 0 = N (N/2 for BLZ_EPI_SWIGLU) */
    float b_scale2;       /* BLZ_EPI_SWIGLU: dequantisation multiplier of the up rows; 0 = b_scale */
    int32_t flags;        /* blz_gemm_flags, 0 = defaults */
} blz_gemm_desc;

typedef struct blz_plan_info {
    int32_t variant;          /* blz_variant actually used */
    int32_t tile_m, tile_n;   /* output tile of one CTA */
    int32_t stages;           /* shared-memory pipeline depth */
    int32_t split_k;          /* 1 unless the decode variant splits K */
    int32_t grid;             /* CTAs launched */
    int32_t smem_bytes;       /* dynamic shared memory per CTA */
    int32_t tmem_cols;        /* tensor-memory columns per CTA */
    int32_t launches;         /* kernels one blz_gemm_execute launches */
    int32_t scheduler;        /* 0 = static persistent schedule, 1 = cluster launch control */
    int64_t workspace_bytes;  /* device memory the plan owns */
    int32_t tail_tiles;       /* tiles that are cut along K (BLZ_FLAG_TAIL_SPLIT; 0 = none), and */
    int32_t tail_split;       /* ... into how many units each */
} blz_plan_info;

typedef struct blz_gemm_plan blz_gemm_plan;

/* Version of this ABI (increments on incompatible change). */
int blz_version(void);
const char* blz_status_string(blz_status s);
/* cudaError_t / CUresult of the last failed CUDA call on this thread, and its text. */
int blz_last_cuda_error(void);
const char* blz_last_cuda_error_string(void);

/* Builds everything one GEMM needs ahead of time: operand repacking for the layouts above,
 * tensor maps, workspace, kernel choice.  Uses the current device; synchronises the device
 * before returning.  The operand pointers in `desc` must stay valid while the plan lives. */
blz_status blz_gemm_plan_create(const blz_gemm_desc* desc, blz_gemm_plan** out_plan);

/* Launches the planned GEMM into C ([M, ldc], the plan's output type).  Asynchronous on `stream`,
 * allocates nothing.  One plan must not run on two streams at the same time. */
blz_status blz_gemm_execute(blz_gemm_plan* plan, void* C, void* stream);

/* Rebinds the A operand (same shape, dtype and scale layout; NVFP4 scales must be BLZ_SF_TILED)
 * without touching anything else.  Host-side only: re-encodes one tensor map. */
blz_status blz_gemm_plan_set_a(blz_gemm_plan* plan, const void* A, const void* A_sf, float a_scale);

/* Synchronises `stream` and reports BLZ_ERR_DEVICE_TIMEOUT if any launch of this plan gave up
 * on a device-side wait since the last check (the error word is cleared). */
blz_status blz_gemm_plan_check(blz_gemm_plan* plan, void* stream);

blz_status blz_gemm_plan_info(const blz_gemm_plan* plan, blz_plan_info* info);

/* Brings everything the plan derived from the weights at creation up to date (asynchronous on `stream`): the
 * K-major copy of [K, N] weights, the tiled copy of row-major scales, the 16-bit copy of BLZ_FLAG_STATIC_WEIGHTS
 * plans.  Call it after B or B_sf changed in place.  Nothing to do, BLZ_OK, for plans that read the caller's
 * K-major weights and tiled scales directly. */
blz_status blz_gemm_plan_refresh_weights(blz_gemm_plan* plan, void* stream);

/* Frees the plan and what it owns.  Null is accepted. */
blz_status blz_gemm_plan_destroy(blz_gemm_plan* plan);

/* plan_create + execute + stream sync + destroy, for callers that run a shape once. */
blz_status blz_gemm_launch(const blz_gemm_desc* desc, void* C, void* stream);

/* ---- operand preparation (device kernels, asynchronous on `stream`) ---- */

/* |x| maximum of n values into *d_amax (device float; combined with its previous content, so
 * zero it first).  x_dtype: BLZ_F32, BLZ_F16 or BLZ_BF16. */
blz_status blz_amax(const void* x, int32_t x_dtype, int64_t n, float* d_amax, void* stream);

/* Per-tensor E4M3 quantisation: s = 448 / *d_amax (1 if amax is 0); q = e4m3_rn(x * s);
 * writes the dequantisation multiplier 1/s ... as two floats d_scales[0] = s, d_scales[1] = 1/s. */
blz_status blz_quantize_fp8(const void* x, int32_t x_dtype, int64_t n, const float* d_amax,
                            uint8_t* q, float* d_scales, void* stream);

/* Two-level NVFP4 quantisation of a [rows, K] row-major matrix, K a multiple of 16:
 *   g = *d_amax / (6*448) (1 if amax is 0); per 16 values along K sf = e4m3_rn((amax_blk/6)/g);
 *   q = e2m1_rn(x / (g*float(sf))), zero when sf is zero.
 * data: [rows, K/2]; sf: row-major [rows, K/16] or tiled (sf_layout), tiled buffers must be
 * blz_tiled_scales_bytes(rows, K) long and are fully written; *d_global = g. */
blz_status blz_quantize_nvfp4(const void* x, int32_t x_dtype, int64_t rows, int64_t K, const float* d_amax,
                              uint8_t* data, uint8_t* sf, int32_t sf_layout, float* d_global, void* stream);

/* out = groups of `group_bytes` bytes taken alternately from `gate` and `up` (group g of gate, group g
 * of up, group g+1 of gate, ...); n_groups groups from each, group_bytes a multiple of 4.  Builds the
 * interleaved weights of BLZ_EPI_SWIGLU from two separate tensors:
 *   K-major packed E2M1 [N_out, K/2]:  n_groups = N_out/16, group_bytes = 16*K/2
 *   row-major scales [N_out, K/16]:    n_groups = N_out/16, group_bytes = 16*K/16
 *   Blaze's [K, N_out/2] packed data:  n_groups = K*N_out/16, group_bytes = 8
 *   Blaze's [K/16, N_out] scales:      n_groups = (K/16)*N_out/16, group_bytes = 16
 *   16-bit or E4M3 K-major weights:    n_groups = N_out/16, group_bytes = 16 * bytes per row */
blz_status blz_interleave_gate_up(const void* gate, const void* up, void* out, int64_t n_groups, int64_t group_bytes, void* stream);

/* Size of the tiled scale-factor array for a [rows, K] operand:
 * ceil(rows/128) row blocks x (ceil(K/64) rounded up to a multiple of 4) atoms x 512 bytes. */
int64_t blz_tiled_scales_bytes(int64_t rows, int64_t K);

/* Row-major E4M3 scales -> tiled.  The scale of (row r, K block b) is read from
 * sf[r*row_stride + b*blk_stride] and written to byte
 *   ((r/128)*katoms + b/4)*512 + (r%32)*16 + ((r%128)/32)*4 + b%4,
 * every other byte of `tiled` is set to zero. */
blz_status blz_tile_scales(const uint8_t* sf, int64_t rows, int64_t K, int64_t row_stride, int64_t blk_stride,
                           uint8_t* tiled, void* stream);

/* ---- bounded-wait self test (no counterpart in the reference, whose waits spin forever:
 *      include/gemm/tma_utils.cuh:217-230) ----
 * Launches one CTA that waits, with the bounded wait every kernel here uses, on a barrier nothing
 * will ever complete; after limit_ns (<= 100 ms) it gives up, sets *d_status non-zero, writes the
 * time it waited to *d_waited_ns (optional) and returns normally.  Shows, without faulting or
 * hanging anything, that a lost arrival becomes an error word instead of a hung GPU. */
blz_status blz_wait_probe(uint64_t limit_ns, int32_t* d_status, uint64_t* d_waited_ns, void* stream);

/* ---- several GPUs: fused GEMM + all-gather (no counterpart in the reference, which has no
 *      multi-GPU code; the sharded benchmark configuration gathers the bf16 output with NCCL after the GEMM) ----
 *
 * Peer-visible buffers: blz_peer_buffer_create allocates device memory and returns a 64-byte
 * CUDA IPC handle; another process of the same box opens it with blz_peer_buffer_open (peer
 * access is enabled lazily) and gets a pointer it may pass as a destination below.
 *
 * blz_gemm_execute_gather runs the planned GEMM (M x N_local x K, tiled variants only) and
 * stores its [M, N_local] block at columns [col_offset, col_offset + N_local) of EVERY
 * destination: dst[i] is the base of the full [M, ld_total] output on GPU i (the caller's own
 * buffer included).  The epilogue writes each staged chunk once per destination with TMA stores,
 * so NVLink traffic overlaps the main loop; when every rank has run it and the ranks have met at
 * a barrier, every GPU holds the whole [M, N_total] matrix in row-major order.  ld_total and
 * col_offset in elements; all bases 16-byte aligned, col_offset a multiple of 8; n_dst <= 8;
 * residual-add epilogues are not supported here. */
blz_status blz_peer_buffer_create(int64_t bytes, void** ptr, uint8_t* handle64);
blz_status blz_peer_buffer_open(const uint8_t* handle64, void** ptr);
blz_status blz_peer_buffer_close(void* ptr);
blz_status blz_peer_buffer_destroy(void* ptr);
blz_status blz_gemm_execute_gather(blz_gemm_plan* plan, int32_t n_dst, void* const* dst, int64_t ld_total,
                                   int64_t col_offset, void* stream);

/* ---- column-sharded GEMM across the GPUs of one box (no counterpart in the reference, which has no multi-GPU
 *      code; the plan triple follows its create / execute / destroy plans,
 *      include/gemm/fp4_blkscaled_gemm_sm100.cuh:198-208) ----
 *
 * Output columns are independent: rank r of `world` owns columns [lo, hi) = blz_shard_bounds(N, world, r, 128)
 * -- rows [lo, hi) of the K-major weights and of their scales -- activations are replicated, and every rank
 * runs the ordinary single-GPU plan on (M, hi - lo, K).  One process per GPU; each process creates its own
 * sharded plan with the device it computes on current.  What follows the GEMM is chosen by `exchange`:
 *
 *   BLZ_EXCHANGE_NONE         nothing: execute writes this rank's [M, hi - lo] block to C
 *   BLZ_EXCHANGE_NCCL         ncclAllGather of the blocks: execute writes [world][M][hi - lo] to C.  NCCL is
 *                             loaded at run time (libnccl.so.2, or BLZ_NCCL_LIBRARY); rank 0 makes an id with
 *                             blz_nccl_unique_id, every rank passes the same 128 bytes in desc.nccl_id, and
 *                             plan creation is collective (ncclCommInitRank)
 *   BLZ_EXCHANGE_PEER_STORES  fused into the GEMM: the plan owns a peer-visible row-major [M, N] output; after
 *                             creation every rank publishes blz_sharded_plan_output_handle (64 bytes), collects
 *                             all ranks' handles in rank order and calls blz_sharded_plan_connect; execute then
 *                             stores every tile into every rank's output (C is ignored).  The ranks must meet at
 *                             a barrier of their own before reading the output or reusing it.
 *
 * desc.gemm describes the FULL problem (N = all columns) with B / B_sf pointing at THIS RANK's rows of the
 * K-major weights (row-major scales: its rows; tiled scales: tiled for the shard); residual-add and the fused
 * gate / up epilogue are not supported here. */
typedef enum blz_exchange { BLZ_EXCHANGE_NONE = 0, BLZ_EXCHANGE_NCCL = 1, BLZ_EXCHANGE_PEER_STORES = 2 } blz_exchange;

typedef struct blz_sharded_desc {
    blz_gemm_desc gemm;      /* see above */
    int32_t world, rank;     /* 1 <= world <= 8 */
    int32_t exchange;        /* blz_exchange */
    int32_t reserved;        /* set to 0 */
    const uint8_t* nccl_id;  /* BLZ_EXCHANGE_NCCL with world > 1: 128 bytes from blz_nccl_unique_id */
} blz_sharded_desc;

typedef struct blz_sharded_info {
    int64_t col_lo, col_hi;  /* output columns of this rank */
    int32_t exchange, world, rank, reserved;
    void* own_output;        /* BLZ_EXCHANGE_PEER_STORES: this rank's [M, N] output (device pointer), else null */
    blz_plan_info gemm;      /* the local plan */
} blz_sharded_info;

typedef struct blz_sharded_plan blz_sharded_plan;

/* Host arithmetic only (no device needed): equal shards of whole `multiple`-column tiles, or
 * BLZ_ERR_INVALID_ARGUMENT when N does not split that way. */
blz_status blz_shard_bounds(int64_t n_total, int32_t world, int32_t rank, int32_t multiple, int64_t* lo, int64_t* hi);
blz_status blz_nccl_unique_id(uint8_t* id128);
blz_status blz_sharded_plan_create(const blz_sharded_desc* desc, blz_sharded_plan** out_plan);
blz_status blz_sharded_plan_info(const blz_sharded_plan* plan, blz_sharded_info* info);
blz_status blz_sharded_plan_output_handle(blz_sharded_plan* plan, uint8_t* handle64);
blz_status blz_sharded_plan_connect(blz_sharded_plan* plan, const uint8_t* handles /* world x 64 bytes, rank order */);
blz_status blz_sharded_plan_execute(blz_sharded_plan* plan, void* C, void* stream);
blz_status blz_sharded_plan_check(blz_sharded_plan* plan, void* stream);
blz_status blz_sharded_plan_destroy(blz_sharded_plan* plan);
/* text of the last NCCL-side failure on this thread */
const char* blz_sharded_last_error(void);

/* ---- allocation-free entry point (no counterpart in the reference: Blaze's launchers and plans
 *      all call cudaMalloc, e.g. src/kernels/gemm_fp4_blkscaled_sm100.cu:840-920) ----
 *
 * The skinny-M NVFP4 GEMM (M <= 64) for callers that must not allocate device memory: serving
 * runtimes that gave all of HBM to their own arena at start-up, and loops that cannot afford an
 * allocation's implicit synchronisation.  It runs a split-K kernel of its own (partial sums in
 * global memory, the last CTA to arrive at a tile adds them in split order) whose workspace is a
 * fixed array inside the library image (8 MiB + 8 KiB per GPU, held by every GPU that loads the
 * library until the process exits) instead of plan-owned memory.  It cuts K exactly as a plan with
 * BLZ_VARIANT_DECODE does and adds the splits in the same order, so the two give bit-identical
 * results.  The call performs no cudaMalloc / cudaFree and uses no allocating library routine.
 *
 *   A, A_sf_tiled : activations, packed E2M1 [M, K/2] and their scales in the TILED layout
 *   B, B_sf_tiled : weights, packed E2M1 [N, K/2] (K-major) and their TILED scales
 *   C             : [M, ldc] of out_dtype (ldc 0 = N); no bias / activation / residual
 *   d_status      : optional device int the kernel sets non-zero if it gives up on a bounded
 *                   wait (caller clears and reads it).  With a null pointer such a give-up is
 *                   NOT reported: the word then goes to the shared array and the next call clears it
 *
 * Limits: M <= 64; ceil(N/128) <= 1024; split * rows * ceil(N/128)*128 * 4 bytes of partial sums
 * <= 8 MiB (rows = 16, 32 or 64 for M <= 16, 32, 64).  Anything larger returns
 * BLZ_ERR_TOO_LARGE and launches nothing.
 * The first call on each device resolves the array's device address and raises the kernels'
 * shared-memory limit (with that device current); make that first call before any stream capture.
 * That first call is also when the driver loads the module that contains the array, i.e. when the
 * 8 MiB are taken from device memory: a caller whose arena claims all free memory must make one
 * call per device (any small shape) BEFORE it sizes the arena; if the memory is already gone the
 * call returns BLZ_ERR_OUT_OF_MEMORY.  Later calls leave the device's free memory untouched.
 * All calls on a device share the one array: the tile counters are cleared at the start of each
 * call, and two calls whose kernels overlap on the GPU (different streams) race on it. */
blz_status blz_gemm_nvfp4_decode_static(const void* A, const void* A_sf_tiled, float a_scale,
                                        const void* B, const void* B_sf_tiled, float b_scale,
                                        int32_t M, int32_t N, int32_t K, void* C, int32_t out_dtype, int64_t ldc,
                                        int32_t* d_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BLAZE_B200_H */
