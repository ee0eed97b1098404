// capi.cu -- implementation of the C ABI declared in include/blaze_b200.h: plan construction
// (operand repacking, tensor maps, kernel choice), launches, and the operand-preparation calls.
//
// Counterpart of the host halves of Blaze's src/kernels/gemm_*_sm100.cu (launch_* and
// create_/execute_/destroy_ plans, e.g. gemm_fp8_sm100.cu:268-430,
// gemm_fp4_blkscaled_sm100.cu:708-951,1083-1230).  Unlike those, nothing here exits the process:
// every failure is a status code, and the device-side error word is read by blz_gemm_plan_check.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <type_traits>

#define BLZ_TUNING_ENTRY_POINTS        // tuning builds only: this translation unit carries the counter read-back calls
#include "../../include/blaze_b200.h"
#include "decode_split.h"
#include "decode_stream_kernel.cuh"
#include "gemm_cluster_kernel.cuh"
#include "prep_kernels.cuh"

using namespace blz;

namespace {

thread_local int g_last_cuda_error = 0;
thread_local char g_last_cuda_error_text[256] = "";

bool cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    g_last_cuda_error = static_cast<int>(e);
    snprintf(g_last_cuda_error_text, sizeof(g_last_cuda_error_text), "%s: %s", what, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return false;
}
#define BLZ_CUDA(call)                                             \
    do {                                                           \
        if (!cuda_ok((call), #call)) return BLZ_ERR_CUDA;          \
    } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so the library has no link-time dependency on
// libcuda and can be loaded (not run) on a machine without a GPU driver.
EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// 2-D byte-typed tensor map over a row-major matrix: `inner_bytes` contiguous bytes per row,
// `rows` rows, `pitch_bytes` apart; box = box_inner bytes x box_rows rows.
blz_status encode_map(CUtensorMap* m, const void* base, uint64_t inner_bytes, uint64_t rows, uint64_t pitch_bytes,
                      uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        snprintf(g_last_cuda_error_text, sizeof(g_last_cuda_error_text), "cuTensorMapEncodeTiled entry point not found");
        return BLZ_ERR_CUDA;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (pitch_bytes & 15u) != 0) return BLZ_ERR_INVALID_ARGUMENT;
    cuuint64_t dims[2] = {inner_bytes, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = static_cast<int>(r);
        snprintf(g_last_cuda_error_text, sizeof(g_last_cuda_error_text), "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
        return BLZ_ERR_CUDA;
    }
    return BLZ_OK;
}

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

int64_t sf_katoms(int64_t K) { return round_up(ceil_div(K, 64), 4); }
int64_t sf_row_blocks(int64_t rows) { return round_up(ceil_div(rows, 128), 2); }

int elem_bytes_out(int dt) { return dt == BLZ_F32 ? 4 : 2; }

int grid_for(int64_t work_items, int threads) {
    int64_t g = ceil_div(work_items, threads);
    if (g < 1) g = 1;
    if (g > 148 * 16) g = 148 * 16;
    return static_cast<int>(g);
}

struct ClusterChoice {
    const void* fn;
    int cg, bn, stages, acc_bufs, smem, tmem_cols, threads, share, epi_warps;
};

template <int KIND, int CG, int BN, int STAGES, int ACC, int SHARE = 1, bool TAIL = false>
ClusterChoice cluster_choice() {
    using Cfg = ClusterGemmConfig<KIND, CG, BN, STAGES, ACC, SHARE>;
    return ClusterChoice{reinterpret_cast<const void*>(&gemm_cluster_kernel<KIND, CG, BN, STAGES, ACC, SHARE, TAIL>), CG, BN, STAGES, ACC,
                         static_cast<int>(Cfg::SMEM_BYTES), static_cast<int>(Cfg::TMEM_COLS), Cfg::THREADS, SHARE, 4 * Cfg::EPI_SETS};
}

// the instances that can run K-split units of the tail (BLZ_FLAG_TAIL_SPLIT): 128x128 and 256x256 tiles of the three
// tensor-core kinds
ClusterChoice pick_tail_kernel(int mma_kind, int cg) {
    if (cg == 2) {
        switch (mma_kind) {
            case MMA_F16: return cluster_choice<MMA_F16, 2, 256, 6, 2, 1, true>();
            case MMA_F8: return cluster_choice<MMA_F8, 2, 256, 6, 2, 1, true>();
            default: return cluster_choice<MMA_NVF4, 2, 256, 5, 1, 1, true>();
        }
    }
    switch (mma_kind) {
        case MMA_F16: return cluster_choice<MMA_F16, 1, 128, 6, 2, 1, true>();
        case MMA_F8: return cluster_choice<MMA_F8, 1, 128, 6, 2, 1, true>();
        default: return cluster_choice<MMA_NVF4, 1, 128, 5, 2, 1, true>();
    }
}

ClusterChoice pick_cluster_kernel(int mma_kind, int cg, int share, bool wide = false, bool narrow = false) {
    if (wide) return cluster_choice<MMA_NVF4, 2, 384, 4, 1>();
    if (narrow) {       // CTA pairs on 256x128 tiles: 24 KB per stage, eight stages, two accumulators
        switch (mma_kind) {
            case MMA_F16: return cluster_choice<MMA_F16, 2, 128, 8, 2>();
            case MMA_F8: return cluster_choice<MMA_F8, 2, 128, 8, 2>();
            default: return cluster_choice<MMA_NVF4, 2, 128, 6, 2>();
        }
    }
    if (cg == 2 && share == 2) {
        switch (mma_kind) {
            case MMA_F16: return cluster_choice<MMA_F16, 2, 256, 6, 2, 2>();
            case MMA_F8: return cluster_choice<MMA_F8, 2, 256, 6, 2, 2>();
            default: return cluster_choice<MMA_NVF4, 2, 256, 5, 1, 2>();
        }
    }
    if (cg == 2) {
        switch (mma_kind) {
            case MMA_W4A16: return cluster_choice<MMA_W4A16, 2, 256, 5, 2>();
            case MMA_F16: return cluster_choice<MMA_F16, 2, 256, 6, 2>();
            case MMA_F8: return cluster_choice<MMA_F8, 2, 256, 6, 2>();
            default: return cluster_choice<MMA_NVF4, 2, 256, 5, 1>();
        }
    }
    switch (mma_kind) {
        case MMA_W4A16: return cluster_choice<MMA_W4A16, 1, 128, 5, 2>();
        case MMA_F16: return cluster_choice<MMA_F16, 1, 128, 6, 2>();
        case MMA_F8: return cluster_choice<MMA_F8, 1, 128, 6, 2>();
        default: return cluster_choice<MMA_NVF4, 1, 128, 5, 2>();
    }
}

}  // namespace

struct blz_gemm_plan {
    blz_gemm_desc desc;
    int device = 0, num_sms = 0;
    int mma_kind = 0;
    int variant = 0;
    // operands as the kernels consume them (K-major, tiled scales)
    const void* a_used = nullptr;
    const void* b_used = nullptr;
    const uint8_t* sfa_used = nullptr;
    const uint8_t* sfb_used = nullptr;
    // device memory the plan owns
    void* own_b = nullptr;
    void* own_sfa = nullptr;
    void* own_sfb = nullptr;
    void* own_w16 = nullptr;      // W4A16: weights expanded to 16 bit, refreshed by every execute -- or only at creation
    bool w16_static = false;      //   (BLZ_FLAG_STATIC_WEIGHTS)
    float* own_tail = nullptr;    // split tail of the schedule: fp32 partial sums of the K-split units, [units][tile rows][BN] in all
    uint32_t* tail_flags = nullptr;   //   and one arrival counter per tail tile and CTA of a group
    uint32_t tail_seq = 0;        //   launches that ran the split tail so far (the counters only grow)
    int tail_tiles = 0, tail_split = 1, tail_first = 0, tail_kps = 0;
    float* own_partial = nullptr; // split-K of the tiled kernel: [splits][m_tiles*128][partial_pitch] fp32
    int split_k = 1;
    int64_t partial_pitch = 0, partial_rows = 0;
    int* status = nullptr;
    int64_t owned_bytes = 0;
    CUtensorMap tm_a{}, tm_b{};
    int grid = 0;
    // cluster-kernel launch (CTA groups of 1 or 2)
    ClusterChoice cc{};
    ClusterGemmParams cp{};
    OutputMaps out{};
    const void* out_ptr[BLZ_MAX_DST] = {};   // what the cached output maps were encoded for
    int64_t out_ld = 0;
    int out_n = 0;
    // decode-kernel launch
    DecodeStreamParams dp{};
    int decode_smem = 0, decode_stages = 0, decode_split = 1, decode_mma_n = 0, decode_tmem = 0, decode_threads = 0;
    const void* decode_fn = nullptr;
    int launches = 1;
    int clc = 0;
};

namespace {

blz_status dev_alloc(blz_gemm_plan* p, void** out, int64_t bytes, bool zero) {
    if (!cuda_ok(cudaMalloc(out, static_cast<size_t>(bytes)), "cudaMalloc")) return BLZ_ERR_OUT_OF_MEMORY;
    p->owned_bytes += bytes;
    if (zero) BLZ_CUDA(cudaMemset(*out, 0, static_cast<size_t>(bytes)));
    return BLZ_OK;
}

blz_status validate(const blz_gemm_desc* d) {
    if (!d) return BLZ_ERR_INVALID_ARGUMENT;
    if (d->M <= 0 || d->N <= 0 || d->K <= 0) return BLZ_ERR_INVALID_ARGUMENT;
    if (!d->A || !d->B) return BLZ_ERR_INVALID_ARGUMENT;
    if (d->kind < BLZ_GEMM_F16 || d->kind > BLZ_GEMM_W4A16_BF16) return BLZ_ERR_INVALID_ARGUMENT;
    if (d->out_dtype < BLZ_F16 || d->out_dtype > BLZ_F32) return BLZ_ERR_INVALID_ARGUMENT;
    if (d->epilogue < BLZ_EPI_NONE || d->epilogue > BLZ_EPI_SWIGLU) return BLZ_ERR_INVALID_ARGUMENT;
    if (d->epilogue == BLZ_EPI_SWIGLU) {
        // gate / up rows interleaved in groups of 16; C is [M, N/2]
        if (d->N % 32) return BLZ_ERR_INVALID_ARGUMENT;
        if (d->ldc != 0 && d->ldc < d->N / 2) return BLZ_ERR_INVALID_ARGUMENT;
    } else if (d->ldc != 0 && d->ldc < d->N) return BLZ_ERR_INVALID_ARGUMENT;
    const bool fp4_a = d->kind == BLZ_GEMM_NVFP4;
    const bool fp4_b = d->kind == BLZ_GEMM_NVFP4 || d->kind == BLZ_GEMM_W4A16_F16 || d->kind == BLZ_GEMM_W4A16_BF16;
    if (fp4_a && !d->A_sf) return BLZ_ERR_INVALID_ARGUMENT;
    if (fp4_b && !d->B_sf) return BLZ_ERR_INVALID_ARGUMENT;
    // row pitches must be multiples of 16 bytes for the tensor maps
    if (d->kind == BLZ_GEMM_F16 || d->kind == BLZ_GEMM_BF16) { if (d->K % 8) return BLZ_ERR_INVALID_ARGUMENT; }
    else if (d->kind == BLZ_GEMM_FP8) { if (d->K % 16) return BLZ_ERR_INVALID_ARGUMENT; }
    else { if (d->K % 32) return BLZ_ERR_INVALID_ARGUMENT; }
    if (d->b_layout == BLZ_B_NMAJOR && fp4_b && (d->N % 2)) return BLZ_ERR_INVALID_ARGUMENT;
    if ((d->epilogue == BLZ_EPI_BIAS || d->epilogue == BLZ_EPI_BIAS_SILU) && !d->bias) return BLZ_ERR_INVALID_ARGUMENT;
    if (d->epilogue == BLZ_EPI_RESIDUAL_ADD && !d->residual) return BLZ_ERR_INVALID_ARGUMENT;
    return BLZ_OK;
}

// Fills the plan-owned copies of B: K-major data from Blaze's [K, N] convention, tiled scales from row-major ones.
blz_status convert_b(blz_gemm_plan* p, cudaStream_t stream) {
    const blz_gemm_desc& d = p->desc;
    const bool fp4_b = d.kind == BLZ_GEMM_NVFP4 || d.kind == BLZ_GEMM_W4A16_F16 || d.kind == BLZ_GEMM_W4A16_BF16;
    const int64_t N = d.N, K = d.K;
    if (p->own_b) {
        if (fp4_b) {
            repack_fp4_kn_to_nk_kernel<<<grid_for((N / 2) * (K / 2), 256), 256, 0, stream>>>(static_cast<const uint8_t*>(d.B), static_cast<uint8_t*>(p->own_b),
                                                                                              static_cast<int>(K), static_cast<int>(N));
        } else {
            dim3 grid(static_cast<unsigned>(ceil_div(N, 32)), static_cast<unsigned>(ceil_div(K, 32))), block(32, 8);
            if (d.kind == BLZ_GEMM_FP8) transpose_kn_to_nk_kernel<uint8_t><<<grid, block, 0, stream>>>(static_cast<const uint8_t*>(d.B), static_cast<uint8_t*>(p->own_b), static_cast<int>(K), static_cast<int>(N));
            else transpose_kn_to_nk_kernel<uint16_t><<<grid, block, 0, stream>>>(static_cast<const uint16_t*>(d.B), static_cast<uint16_t*>(p->own_b), static_cast<int>(K), static_cast<int>(N));
        }
        BLZ_CUDA(cudaGetLastError());
    }
    if (p->own_sfb) {
        BLZ_CUDA(cudaMemsetAsync(p->own_sfb, 0, static_cast<size_t>(blz_tiled_scales_bytes(N, K)), stream));
        const int64_t kb = K / 16;
        const int64_t row_stride = d.b_layout == BLZ_B_NMAJOR ? 1 : kb;
        const int64_t blk_stride = d.b_layout == BLZ_B_NMAJOR ? N : 1;
        tile_scales_kernel<<<grid_for(N * kb, 256), 256, 0, stream>>>(static_cast<const uint8_t*>(d.B_sf), N, kb, row_stride, blk_stride, sf_katoms(K),
                                                                      static_cast<uint8_t*>(p->own_sfb));
        BLZ_CUDA(cudaGetLastError());
    }
    return BLZ_OK;
}

// B as the kernels consume it: K-major as is, or a plan-owned K-major copy; scales tiled as is, or a plan-owned tiled copy.
blz_status prepare_b(blz_gemm_plan* p) {
    const blz_gemm_desc& d = p->desc;
    const bool fp4_b = d.kind == BLZ_GEMM_NVFP4 || d.kind == BLZ_GEMM_W4A16_F16 || d.kind == BLZ_GEMM_W4A16_BF16;
    const int64_t N = d.N, K = d.K;
    p->b_used = d.B;
    if (d.b_layout == BLZ_B_NMAJOR) {
        const int64_t bytes = fp4_b ? N * K / 2 : N * K * (d.kind == BLZ_GEMM_FP8 ? 1 : 2);
        blz_status s = dev_alloc(p, &p->own_b, bytes, false);
        if (s) return s;
        p->b_used = p->own_b;
    }
    if (fp4_b) {
        if (d.b_sf_layout == BLZ_SF_TILED && d.b_layout == BLZ_B_KMAJOR) {
            p->sfb_used = static_cast<const uint8_t*>(d.B_sf);
        } else {
            blz_status s = dev_alloc(p, &p->own_sfb, blz_tiled_scales_bytes(N, K), false);
            if (s) return s;
            p->sfb_used = static_cast<const uint8_t*>(p->own_sfb);
        }
    }
    return convert_b(p, nullptr);
}

blz_status prepare_a_scales(blz_gemm_plan* p) {
    const blz_gemm_desc& d = p->desc;
    if (d.kind != BLZ_GEMM_NVFP4) return BLZ_OK;
    if (d.a_sf_layout == BLZ_SF_TILED) { p->sfa_used = static_cast<const uint8_t*>(d.A_sf); return BLZ_OK; }
    const int64_t bytes = blz_tiled_scales_bytes(d.M, d.K);
    blz_status s = dev_alloc(p, &p->own_sfa, bytes, true);
    if (s) return s;
    const int64_t kb = d.K / 16;
    tile_scales_kernel<<<grid_for(static_cast<int64_t>(d.M) * kb, 256), 256>>>(static_cast<const uint8_t*>(d.A_sf), d.M, kb, kb, 1, sf_katoms(d.K),
                                                                                static_cast<uint8_t*>(p->own_sfa));
    BLZ_CUDA(cudaGetLastError());
    p->sfa_used = static_cast<const uint8_t*>(p->own_sfa);
    return BLZ_OK;
}

// bytes of one operand row as the tensor core reads it
int64_t row_bytes(int mma_kind, int64_t K) { return mma_kind == MMA_F16 ? K * 2 : mma_kind == MMA_F8 ? K : K / 2; }

int env_int(const char* name, int fallback);

blz_status launch_config_cluster(const blz_gemm_plan* p, cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, cudaStream_t stream) {
    cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p->grid));
    cfg.blockDim = dim3(static_cast<unsigned>(p->cc.threads));
    cfg.dynamicSmemBytes = static_cast<size_t>(p->cc.smem);
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(p->cc.cg * p->cc.share);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return BLZ_OK;
}

blz_status setup_cluster(blz_gemm_plan* p, int cg, int share = 1, bool wide = false, bool narrow = false) {
    const blz_gemm_desc& d = p->desc;
    const int64_t rb = row_bytes(p->mma_kind, d.K);
    if (wide && p->mma_kind != MMA_NVF4) return BLZ_ERR_UNSUPPORTED;
    // W4A16 without a 16-bit copy of the weights: the kernel expands the packed weights itself
    const bool fused_w4 = (d.kind == BLZ_GEMM_W4A16_F16 || d.kind == BLZ_GEMM_W4A16_BF16) && p->own_w16 == nullptr;
    if (fused_w4 && (share != 1 || narrow)) return BLZ_ERR_UNSUPPORTED;
    p->cc = pick_cluster_kernel(fused_w4 ? static_cast<int>(MMA_W4A16) : p->mma_kind, cg, share, wide, narrow);
    p->variant = wide ? BLZ_VARIANT_PAIR_256x384 : narrow ? BLZ_VARIANT_PAIR_256x128 : share == 2 ? BLZ_VARIANT_QUAD_512x256 : cg == 2 ? BLZ_VARIANT_PAIR_256x256 : BLZ_VARIANT_TILE_128x128;
    BLZ_CUDA(cudaFuncSetAttribute(p->cc.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, p->cc.smem));
    const int bn = p->cc.bn, tile_m = 128 * cg;
    blz_status s = encode_map(&p->tm_a, p->a_used, static_cast<uint64_t>(rb), static_cast<uint64_t>(d.M), static_cast<uint64_t>(rb), 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (s) return s;
    if (fused_w4) {
        // packed weights: 32 bytes (64 K values) x 128 rows per stage, unswizzled -- the expansion warps read them
        const int64_t rbw = d.K / 2;
        s = encode_map(&p->tm_b, p->b_used, static_cast<uint64_t>(rbw), static_cast<uint64_t>(d.N), static_cast<uint64_t>(rbw), 32, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else {
        s = encode_map(&p->tm_b, p->b_used, static_cast<uint64_t>(rb), static_cast<uint64_t>(d.N), static_cast<uint64_t>(rb), 128, wide ? 64u : static_cast<uint32_t>(bn / cg / share), CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (s) return s;
    ClusterGemmParams& cp = p->cp;
    cp.M = d.M; cp.N = d.N;
    cp.m_tiles = static_cast<int>(ceil_div(d.M, tile_m * share));
    cp.n_tiles = static_cast<int>(ceil_div(d.N, bn));
    // Rasterisation: when all of A stays in L2 anyway (it is re-read by every column of tiles),
    // walk M fastest so that concurrent tiles share as few B panels as possible; otherwise cut M
    // into bands of 8 tiles so that one wave of CTA groups covers a near-square block.
    cp.group_m = (static_cast<int64_t>(d.M) * rb <= (48ll << 20)) ? cp.m_tiles : 8;
    cp.group_m = env_int("BLZ_GROUP_M", cp.group_m);
    if (cp.group_m < 1) cp.group_m = 1;
    cp.k_stages = static_cast<int>(ceil_div(rb, 128));
    // Few 128x128 tiles and a long K (decode-like N with a prefill-like M): split K over up to four
    // CTAs per tile.  Split s of M tile m runs as M tile s * m_tiles + m and stores fp32 partial
    // sums to its own row block of a scratch matrix; a small second kernel adds the splits in order
    // and applies the epilogue.
    cp.m_tiles_real = cp.m_tiles; cp.split_k = 1; cp.k_per_split = cp.k_stages;
    if (cg == 1 && share == 1 && !wide && d.epilogue != BLZ_EPI_SWIGLU) {
        int split = 1;
        const int64_t tiles1 = static_cast<int64_t>(cp.m_tiles) * cp.n_tiles;
        while (split < 4 && tiles1 * split * 2 <= p->num_sms && cp.k_stages / (split * 2) >= 16) split *= 2;
        split = env_int("BLZ_TILE_SPLIT_K", split);
        while (split > 1 && (split - 1) * static_cast<int>(ceil_div(cp.k_stages, split)) >= cp.k_stages) --split;   // no empty split
        if (split > 1) {
            p->split_k = split;
            p->partial_rows = static_cast<int64_t>(cp.m_tiles) * 128;
            p->partial_pitch = round_up(d.N, 4);
            void* mem = nullptr;
            blz_status st = dev_alloc(p, &mem, static_cast<int64_t>(split) * p->partial_rows * p->partial_pitch * 4, false);
            if (st) return st;
            p->own_partial = static_cast<float*>(mem);
            cp.split_k = split;
            cp.k_per_split = static_cast<int>(ceil_div(cp.k_stages, split));
            cp.m_tiles = cp.m_tiles_real * split;
            p->launches += 1;
        }
    }
    const uint32_t fmt = d.kind == BLZ_GEMM_BF16 || d.kind == BLZ_GEMM_W4A16_BF16 ? 1u : 0u;
    cp.idesc2 = make_idesc_nvf4(tile_m, 128);
    cp.sfb_row_blocks = static_cast<int>(sf_row_blocks(d.N));
    cp.expand_bf16 = d.kind == BLZ_GEMM_W4A16_BF16 ? 1 : 0;
    cp.idesc = wide ? make_idesc_nvf4(tile_m, 256) : p->mma_kind == MMA_NVF4 ? make_idesc_nvf4(tile_m, bn) : p->mma_kind == MMA_F8 ? make_idesc(0, 0, tile_m, bn) : make_idesc(fmt, fmt, tile_m, bn);
    cp.sfa = p->sfa_used; cp.sfb = p->sfb_used;
    cp.sf_katoms = static_cast<int>(sf_katoms(d.K));
    cp.status = p->status;
    const int64_t tiles = static_cast<int64_t>(cp.m_tiles) * cp.n_tiles;
    const int csize = cg * share;
    int max_groups = p->num_sms / csize;
    if (csize > 1) {
        // how many pairs the device can hold at once (GPC shapes can leave SMs unpaired)
        p->grid = max_groups * csize;
        cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[1];
        launch_config_cluster(p, cfg, attr, nullptr);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, p->cc.fn, &cfg) == cudaSuccess && n > 0) { if (n < max_groups) max_groups = n; }
        else (void)cudaGetLastError();
    }
    const int64_t groups = tiles < max_groups ? tiles : max_groups;
    p->grid = static_cast<int>(groups) * csize;
    // The tail of the schedule: when the last wave holds at most half as many tiles as there are CTA groups, its
    // tiles can be cut along K so that every group works until the end (4096^3 FP8: 256 tiles on 74 pairs are
    // 3 full waves + 34 tiles -> 68 half-K units; 512 x 12288 x 4096: 74 + 22 tiles -> 66 units of a third of K;
    // 512 x 4096 x 11008: 32 tiles -> 64 units, no whole tile at all).  The units of a tile exchange fp32 partial
    // sums through a plan-owned scratch array inside the same launch and each finishes a slice of the tile's
    // columns (sums in unit order: results do not depend on timing).  Not with the variants whose roles walk a
    // fixed sequence, the fused gate / up epilogue, the tiled kernel's own K split or the launch-queue scheduler.
    // Measured on B200 (per-phase cycle stamps of the tuning build, FP8 4096^3): a unit's exchange -- accumulator
    // to scratch 3.7 k cycles, fence and publish 2.2 k, wait for the other units 1.4 k, sum / finish / store 9 k --
    // costs about as much as 32 K stages of a whole 256x256 tile, so cutting pays only for long K and three or
    // more units (f16 512 x 12288 x 4096: 59.0 -> 55.1 us; FP8 4096^3: 56.0 -> 58.3 us; NVFP4 8192 x 3584 x 8192:
    // 111.3 -> 115.5 us).  It therefore runs on request only: desc.flags & BLZ_FLAG_TAIL_SPLIT, or BLZ_TAIL_SPLIT=1.
    cp.tail_first = static_cast<int>(tiles); cp.tail_split = 1; cp.tail_kps = cp.k_stages; cp.total_units = static_cast<int>(tiles);
    cp.tail_scratch = nullptr; cp.tail_flags = nullptr; cp.tail_target = 0;
    p->tail_tiles = 0; p->tail_split = 1;
    const int64_t tail = tiles % max_groups;
    if (share == 1 && !fused_w4 && !wide && !narrow && cp.split_k == 1 && d.epilogue != BLZ_EPI_SWIGLU && tail > 0 &&
        env_int("BLZ_TAIL_SPLIT", (d.flags & BLZ_FLAG_TAIL_SPLIT) ? 1 : 0) != 0) {
        int split = static_cast<int>(max_groups / tail);
        if (split > 16) split = 16;
        while (split > 1 && cp.k_stages / split < 4) --split;                      // at least four K stages per unit
        int kps = cp.k_stages;
        if (split >= 2) {
            kps = static_cast<int>(ceil_div(cp.k_stages, split));
            split = static_cast<int>(ceil_div(cp.k_stages, kps));                  // no empty unit
        }
        if (split >= 2) {
            const int64_t units = tail * split;
            const int64_t tile_rows = tile_m * share;
            void* mem = nullptr;
            blz_status st = dev_alloc(p, &mem, units * tile_rows * bn * 4, false);
            if (st) return st;
            p->own_tail = static_cast<float*>(mem);
            st = dev_alloc(p, &mem, tail * csize * 4, true);
            if (st) return st;
            p->tail_flags = static_cast<uint32_t*>(mem);
            p->tail_seq = 0;
            p->tail_tiles = static_cast<int>(tail); p->tail_split = split; p->tail_first = static_cast<int>(tiles - tail); p->tail_kps = kps;
            cp.tail_first = p->tail_first; cp.tail_split = split; cp.tail_kps = kps; cp.total_units = static_cast<int>(tiles - tail + units);
            cp.tail_scratch = reinterpret_cast<float4*>(p->own_tail); cp.tail_flags = p->tail_flags;
            p->grid = static_cast<int>(cp.total_units < max_groups ? cp.total_units : max_groups) * csize;    // few tiles: one group per unit
            p->cc = pick_tail_kernel(p->mma_kind, cg);             // same configuration, the instance that knows units
            BLZ_CUDA(cudaFuncSetAttribute(p->cc.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, p->cc.smem));
        }
    }
    // Dynamic scheduling: one cluster per tile in the grid; clusters that are running take over the tiles of
    // clusters that have not started (cluster launch control).  On request (desc.flags / BLZ_SCHEDULER=clc);
    // not for the variants whose roles walk a fixed tile sequence (B sharing, in-kernel W4A16 expansion).
    const char* sched_env = getenv("BLZ_SCHEDULER");
    bool want_clc = (d.flags & BLZ_FLAG_CLC_SCHEDULER) != 0;
    if (sched_env && *sched_env) want_clc = strcmp(sched_env, "clc") == 0;
    cp.clc = (want_clc && share == 1 && !fused_w4 && tiles * csize <= 0x7FFFFFFF) ? 1 : 0;
    if (cp.clc && p->tail_tiles) {           // the launch queue hands out whole tiles only
        cp.tail_first = static_cast<int>(tiles); cp.tail_split = 1; cp.total_units = static_cast<int>(tiles);
        p->tail_tiles = 0; p->tail_split = 1;
        p->grid = static_cast<int>(groups) * csize;
    }
    if (cp.clc) p->grid = static_cast<int>(tiles) * csize;
    p->clc = cp.clc;
    return BLZ_OK;
}

// Tile shape for BLZ_VARIANT_AUTO (M > 128; below that the decode kernels or 128-row tiles).  Large problems take
// 256x256 pair tiles: fewest L2 bytes per FLOP.  Up to three waves of those, the quantisation of the last wave and
// the drain of the last tile decide, and a small model picks among 256x256, 256x128 (pairs) and 128x128 (single
// CTAs): cost = waves x K stages x the variant's time per stage + its drain, in units of one K stage of a 256x256
// tile.  The per-stage factors and drains are fitted to measurements on B200 (18 shapes with M = 256 ... 1024, three
// kinds): a 256x128 tile takes 0.58 of a 256x256 tile's time (0.50 for NVFP4), a wave of 128x128 tiles 0.68 (0.52);
// the model ranks the variants correctly on all of them, e.g. f16 1024 x 4096 x 11008: 70 us (256x256) against 94
// (128x128, the former choice); f16 512 x 4096 x 11008: 52 (256x128) against 56 / 66.  The larger tile wins ties
// (within 7 %).
int choose_tile_variant(const blz_gemm_plan* p, bool fused_w4) {
    const blz_gemm_desc& d = p->desc;
    const int64_t pairs = p->num_sms / 2;
    const int64_t t256 = ceil_div(d.M, 256) * ceil_div(d.N, 256);
    if (d.M <= 128) return BLZ_VARIANT_TILE_128x128;
    if (fused_w4 || d.epilogue == BLZ_EPI_SWIGLU)      // no 256x128 instance of these: pairs when every pair gets a tile
        return t256 >= pairs ? BLZ_VARIANT_PAIR_256x256 : BLZ_VARIANT_TILE_128x128;
    const int64_t w256 = ceil_div(t256, pairs);
    if (w256 > 3) return BLZ_VARIANT_PAIR_256x256;
    const bool nvf4 = p->mma_kind == MMA_NVF4;
    const double ks = static_cast<double>(ceil_div(row_bytes(p->mma_kind, d.K), 128));
    const double r_narrow = nvf4 ? 0.50 : 0.58, r_single = nvf4 ? 0.52 : 0.68;
    const double c256 = static_cast<double>(w256) * ks + 6.0;
    const double c_narrow = static_cast<double>(ceil_div(ceil_div(d.M, 256) * ceil_div(d.N, 128), pairs)) * ks * r_narrow + 3.0;
    const double c_single = static_cast<double>(ceil_div(ceil_div(d.M, 128) * ceil_div(d.N, 128), static_cast<int64_t>(p->num_sms))) * ks * r_single + 3.0;
    const double best = c256 < c_narrow ? (c256 < c_single ? c256 : c_single) : (c_narrow < c_single ? c_narrow : c_single);
    if (c256 <= 1.07 * best) return BLZ_VARIANT_PAIR_256x256;
    if (c_narrow <= 1.07 * best) return BLZ_VARIANT_PAIR_256x128;
    return BLZ_VARIANT_TILE_128x128;
}

void fill_epilogue(const blz_gemm_plan* p, void* C, EpilogueParams& e) {
    const blz_gemm_desc& d = p->desc;
    e.C = C;
    e.bias = d.bias; e.residual = d.residual;
    e.ldc = d.ldc ? d.ldc : (d.epilogue == BLZ_EPI_SWIGLU ? d.N / 2 : d.N); e.ldr = e.ldc;
    e.alpha = d.a_scale * d.b_scale;
    e.alpha2 = d.a_scale * (d.b_scale2 != 0.0f ? d.b_scale2 : d.b_scale);
    e.mode = d.epilogue;
    e.out_type = d.out_dtype;
    const int eb = elem_bytes_out(d.out_dtype);
    bool vec = (reinterpret_cast<uintptr_t>(C) & 15u) == 0 && ((e.ldc * eb) & 15) == 0;
    if (d.residual) vec = vec && (reinterpret_cast<uintptr_t>(d.residual) & 15u) == 0;
    e.vec_ok = vec ? 1 : 0;
}

// ---- decode variant (M <= 64, every kind)

struct DecodeChoice { const void* fn; int mma_n, stages, smem, threads, max_split, tmem_cols; };

template <int KIND, int MMA_N, int STAGES>
DecodeChoice decode_choice() {
    using Cfg = DecodeStreamConfig<KIND, MMA_N, STAGES>;
    return DecodeChoice{reinterpret_cast<const void*>(&decode_stream_kernel<KIND, MMA_N, STAGES>), MMA_N, STAGES, static_cast<int>(Cfg::SMEM_BYTES),
                        Cfg::THREADS, Cfg::MAX_SPLIT, static_cast<int>(Cfg::TMEM_COLS)};
}
template <bool BF16, int MMA_N, int LSTAGES>
DecodeChoice decode_choice_w4a16() {
    using Cfg = DecodeW4A16Config<MMA_N, LSTAGES>;
    return DecodeChoice{reinterpret_cast<const void*>(&decode_w4a16_kernel<BF16, MMA_N, LSTAGES>), MMA_N, LSTAGES, static_cast<int>(Cfg::SMEM_BYTES),
                        Cfg::THREADS, Cfg::MAX_SPLIT, static_cast<int>(Cfg::TMEM_COLS)};
}
template <int KIND>
DecodeChoice decode_choice_for(int M) {
    if constexpr (KIND != MMA_NVF4) { if (M > 64) return decode_choice<KIND, 128, 5>(); }
    return M <= 16 ? decode_choice<KIND, 16, 5>() : M <= 32 ? decode_choice<KIND, 32, 4>() : decode_choice<KIND, 64, 3>();
}
template <bool BF16, int WSTAGES, int XSLOTS>
DecodeChoice decode_choice_w4a16_wide() {
    using Cfg = DecodeW4A16WideConfig<WSTAGES, XSLOTS>;
    return DecodeChoice{reinterpret_cast<const void*>(&decode_w4a16_wide_kernel<BF16, WSTAGES, XSLOTS>), Cfg::MMA_N, WSTAGES, static_cast<int>(Cfg::SMEM_BYTES),
                        Cfg::THREADS, Cfg::MAX_SPLIT, static_cast<int>(Cfg::TMEM_COLS)};
}
template <bool BF16>
DecodeChoice decode_choice_w4a16_for(int M) {
    if (M > 64) return decode_choice_w4a16_wide<BF16, 3, 4>();
    return M <= 16 ? decode_choice_w4a16<BF16, 16, 6>() : M <= 32 ? decode_choice_w4a16<BF16, 32, 6>() : decode_choice_w4a16<BF16, 64, 3>();
}
// The allocation-free entry point (decode_static.cu) cuts K by decode_max_split() alone: the NVFP4
// stream kernels must support at least that much, or the two paths would partition K differently.
static_assert(DecodeStreamConfig<MMA_NVF4, 16, 5>::MAX_SPLIT >= 8 && DecodeStreamConfig<MMA_NVF4, 32, 4>::MAX_SPLIT >= 4 &&
              DecodeStreamConfig<MMA_NVF4, 64, 3>::MAX_SPLIT >= 2, "decode_max_split() exceeds what the NVFP4 stream kernels hold");

DecodeChoice pick_decode_kernel(int mma_kind, bool w4a16, bool bf16, int M) {
    if (w4a16) return bf16 ? decode_choice_w4a16_for<true>(M) : decode_choice_w4a16_for<false>(M);
    switch (mma_kind) {
        case MMA_F16: return decode_choice_for<MMA_F16>(M);
        case MMA_F8: return decode_choice_for<MMA_F8>(M);
        default: return decode_choice_for<MMA_NVF4>(M);
    }
}

int env_int(const char* name, int fallback) {
    const char* v = getenv(name);
    if (!v || !*v) return fallback;
    return atoi(v);
}

bool is_w4a16(const blz_gemm_desc& d) { return d.kind == BLZ_GEMM_W4A16_F16 || d.kind == BLZ_GEMM_W4A16_BF16; }

blz_status decode_encode_x(blz_gemm_plan* p) {
    const blz_gemm_desc& d = p->desc;
    const int64_t rb = row_bytes(p->mma_kind, d.K);      // W4A16 plans carry MMA_F16: 16-bit activations
    return encode_map(&p->tm_a, p->a_used, static_cast<uint64_t>(rb), static_cast<uint64_t>(d.M), static_cast<uint64_t>(rb), 128,
                      static_cast<uint32_t>(p->decode_mma_n), CU_TENSOR_MAP_SWIZZLE_128B);
}

blz_status decode_setup(blz_gemm_plan* p) {
    const blz_gemm_desc& d = p->desc;
    const bool w4 = is_w4a16(d);
    const DecodeChoice dc = pick_decode_kernel(p->mma_kind, w4, d.kind == BLZ_GEMM_W4A16_BF16, d.M);
    p->decode_fn = dc.fn; p->decode_mma_n = dc.mma_n; p->decode_stages = dc.stages; p->decode_smem = dc.smem;
    p->decode_tmem = dc.tmem_cols; p->decode_threads = dc.threads;
    BLZ_CUDA(cudaFuncSetAttribute(dc.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, dc.smem));
    blz_status s;
    DecodeStreamParams& dp = p->dp;
    if (w4) {
        // packed weights: 128 bytes (256 values) x 128 rows per load stage; the expansion warps undo the swizzle
        const int64_t rbw = d.K / 2;
        s = encode_map(&p->tm_b, p->b_used, static_cast<uint64_t>(rbw), static_cast<uint64_t>(d.N), static_cast<uint64_t>(rbw), 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
        dp.k_stages_total = static_cast<int>(ceil_div(rbw, 128));
    } else {
        const int64_t rb = row_bytes(p->mma_kind, d.K);
        s = encode_map(&p->tm_b, p->b_used, static_cast<uint64_t>(rb), static_cast<uint64_t>(d.N), static_cast<uint64_t>(rb), 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
        dp.k_stages_total = static_cast<int>(ceil_div(rb, 128));
    }
    if (s) return s;
    if ((s = decode_encode_x(p))) return s;

    dp.M = d.M; dp.N = d.N;
    dp.n_tiles = static_cast<int>(ceil_div(d.N, 128));
    const int max_split = decode_max_split(dc.mma_n) < dc.max_split ? decode_max_split(dc.mma_n) : dc.max_split;
    dp.split = decode_pick_split(dp.n_tiles, dp.k_stages_total, p->num_sms, max_split, decode_split_override());
    dp.stages_per_split = static_cast<int>(ceil_div(dp.k_stages_total, dp.split));
    // W4A16, M <= 32: one CTA per SM, so a grid beyond one wave costs a whole second kernel time
    // (22016 x 4096: 172 tiles, 24.6 us).  The CTAs then take several consecutive tiles each, up to what
    // the accumulator columns hold (two for M <= 16): 86 CTAs x 2 tiles, 22.2 us.  Combining this with
    // a K split (58 clusters of 2 x 3 tiles) measured 26.1 us -- the reduction over the cluster runs once
    // per tile -- so the automatic choice never splits; BLZ_DECODE_TILES_PER_CTA with BLZ_DECODE_SPLIT forces both.
    dp.tiles_per_cta = (is_w4a16(d) && dc.mma_n <= 32)
                     ? decode_tiles_per_cta(dp.n_tiles, p->num_sms, dc.mma_n, dp.split, env_int("BLZ_DECODE_TILES_PER_CTA", 0)) : 1;
    const uint32_t fmt16 = d.kind == BLZ_GEMM_BF16 || d.kind == BLZ_GEMM_W4A16_BF16 ? 1u : 0u;
    // operands are swapped: the instruction's A is the weight tile, its B the activations
    dp.idesc = p->mma_kind == MMA_NVF4 ? make_idesc_nvf4(128, static_cast<uint32_t>(dc.mma_n))
             : p->mma_kind == MMA_F8 ? make_idesc(0, 0, 128, static_cast<uint32_t>(dc.mma_n))
                                     : make_idesc(fmt16, fmt16, 128, static_cast<uint32_t>(dc.mma_n));
    dp.sfw = p->sfb_used; dp.sfx = p->sfa_used;
    dp.sf_katoms = static_cast<int>(sf_katoms(d.K));
    // Four more weight stages per CTA go to L2 ahead of the wait for the predecessor grid (measured in a
    // chain of decode GEMMs: FP8 22016 x 4096 17.0 -> 16.4 us, NVFP4 4096 x 11008 9.9 -> 9.6 us; 16 or more
    // compete with the predecessor's own loads and lose 5-15 %).  No gain for W4A16, which is not bound by HBM.
    dp.l2_prefetch = env_int("BLZ_DECODE_L2_PREFETCH", is_w4a16(d) ? 0 : 4);
    if (dp.l2_prefetch < 0) dp.l2_prefetch = 0;
    dp.status = p->status;
    p->decode_split = dp.split;
    p->grid = static_cast<int>(ceil_div(dp.n_tiles, dp.tiles_per_cta)) * dp.split;
    return BLZ_OK;
}

blz_status decode_rebind_a(blz_gemm_plan* p) {
    p->dp.sfx = p->sfa_used;
    return decode_encode_x(p);
}

blz_status decode_launch(blz_gemm_plan* p, void* C, cudaStream_t stream) {
    DecodeStreamParams dp = p->dp;
    fill_epilogue(p, C, dp.epi);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p->grid));
    cfg.blockDim = dim3(static_cast<unsigned>(p->decode_threads));
    cfg.dynamicSmemBytes = static_cast<size_t>(p->decode_smem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    // the K splits of one tile form a cluster (partial sums travel through distributed shared memory)
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = static_cast<unsigned>(dp.split);
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
    // programmatic dependent launch: set-up and weight prefetch overlap the previous kernel's tail
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = env_int("BLZ_DECODE_NO_PDL", 0) ? 0 : 1;
    ++na;
    cfg.attrs = attr;
    cfg.numAttrs = static_cast<unsigned>(na);
    // tm_b maps the weights (the 128-row operand), tm_a the activations
    void* args[3] = {&p->tm_b, &p->tm_a, &dp};
    BLZ_CUDA(cudaLaunchKernelExC(&cfg, p->decode_fn, args));
    return BLZ_OK;
}

// W4A16 with a 16-bit copy of the weights: packed E2M1 x block scale -> fp16 / bf16 (exact), the tensor scale stays in alpha.
blz_status expand_weights(blz_gemm_plan* p, cudaStream_t stream) {
    const blz_gemm_desc& d = p->desc;
    const int64_t blocks16 = static_cast<int64_t>(d.N) * (d.K / 8);     // one thread per 8 values
    if (d.kind == BLZ_GEMM_W4A16_F16)
        dequant_nvfp4_kernel<false><<<grid_for(blocks16, 256), 256, 0, stream>>>(static_cast<const uint8_t*>(p->b_used), p->sfb_used, sf_katoms(d.K), d.N, d.K, static_cast<uint16_t*>(p->own_w16));
    else
        dequant_nvfp4_kernel<true><<<grid_for(blocks16, 256), 256, 0, stream>>>(static_cast<const uint8_t*>(p->b_used), p->sfb_used, sf_katoms(d.K), d.N, d.K, static_cast<uint16_t*>(p->own_w16));
    BLZ_CUDA(cudaGetLastError());
    return BLZ_OK;
}

// Launches the cluster kernel.  `dst` are the bases of n_dst output matrices with row pitch `ld`
// (elements); the tile block goes to columns [col_offset, col_offset + N) of each.
blz_status launch_cluster(blz_gemm_plan* p, int n_dst, void* const* dst, int64_t ld, int64_t col_offset, cudaStream_t stream) {
    const blz_gemm_desc& d = p->desc;
    if (p->own_w16 && !p->w16_static) {
        blz_status s = expand_weights(p, stream);
        if (s) return s;
    }
    const int eb = elem_bytes_out(d.out_dtype);
    ClusterGemmParams cp = p->cp;
    if (p->split_k > 1) {
        // K split: the GEMM kernel writes raw fp32 partial sums of every split into the plan's scratch
        // matrix (its "M" is all splits' row blocks), the second kernel finishes into C.
        if (n_dst != 1) return BLZ_ERR_UNSUPPORTED;
        const int64_t rows_all = p->partial_rows * p->split_k;
        cp.M = static_cast<int>(rows_all);
        cp.epi.C = p->own_partial; cp.epi.bias = nullptr; cp.epi.residual = nullptr;
        cp.epi.ldc = p->partial_pitch; cp.epi.ldr = p->partial_pitch;
        cp.epi.alpha = 1.0f; cp.epi.alpha2 = 1.0f; cp.epi.mode = EPI_NONE; cp.epi.out_type = OUT_F32; cp.epi.vec_ok = 1;
        cp.use_tma_store = 1; cp.n_dst = 1;
        if (p->out_n != -1) {
            blz_status s = encode_map(&p->out.m[0], p->own_partial, static_cast<uint64_t>(d.N) * 4, static_cast<uint64_t>(rows_all),
                                      static_cast<uint64_t>(p->partial_pitch) * 4, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
            if (s) return s;
            p->out_n = -1;                          // the cached map describes the scratch matrix
        }
        cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[1];
        launch_config_cluster(p, cfg, attr, stream);
        void* cargs[4] = {&p->tm_a, &p->tm_b, &p->out, &cp};
        BLZ_CUDA(cudaLaunchKernelExC(&cfg, p->cc.fn, cargs));
        EpilogueParams e;
        e.C = static_cast<uint8_t*>(dst[0]) + col_offset * eb;
        e.bias = d.bias; e.residual = d.residual; e.ldc = ld; e.ldr = ld;
        e.alpha = d.a_scale * d.b_scale; e.alpha2 = e.alpha; e.mode = d.epilogue; e.out_type = d.out_dtype; e.vec_ok = 0;
        const int64_t groups = static_cast<int64_t>(d.M) * ceil_div(d.N, 4);
        splitk_reduce_kernel<<<grid_for(groups, 256), 256, 0, stream>>>(p->own_partial, p->split_k, p->partial_rows, p->partial_pitch, d.M, d.N, e);
        BLZ_CUDA(cudaGetLastError());
        return BLZ_OK;
    }
    cp.epi.C = static_cast<uint8_t*>(dst[0]) + col_offset * eb;
    cp.epi.bias = d.bias; cp.epi.residual = d.residual;
    cp.epi.ldc = ld; cp.epi.ldr = ld;
    cp.epi.alpha = d.a_scale * d.b_scale;
    cp.epi.alpha2 = d.a_scale * (d.b_scale2 != 0.0f ? d.b_scale2 : d.b_scale);
    cp.epi.mode = d.epilogue;
    cp.epi.out_type = d.out_dtype;
    bool vec = ((ld * eb) & 15) == 0 && ((col_offset * eb) & 15) == 0;
    for (int i = 0; i < n_dst; ++i) vec = vec && (reinterpret_cast<uintptr_t>(dst[i]) & 15u) == 0;
    if (d.residual) vec = vec && (reinterpret_cast<uintptr_t>(d.residual) & 15u) == 0;
    cp.epi.vec_ok = vec ? 1 : 0;
    // the fused gate / up epilogue writes half-width rows straight from registers
    cp.use_tma_store = (cp.epi.vec_ok && d.epilogue != BLZ_EPI_SWIGLU) ? 1 : 0;
    cp.n_dst = n_dst;
    if (n_dst > 1 && !cp.use_tma_store) return BLZ_ERR_INVALID_ARGUMENT;   // peer outputs go through TMA stores only
    if (cp.use_tma_store) {
        bool same = p->out_n == n_dst && p->out_ld == ld * 1000003 + col_offset;
        for (int i = 0; same && i < n_dst; ++i) same = p->out_ptr[i] == dst[i];
        if (!same) {
            for (int i = 0; i < n_dst; ++i) {
                blz_status s = encode_map(&p->out.m[i], static_cast<uint8_t*>(dst[i]) + col_offset * eb, static_cast<uint64_t>(d.N) * eb,
                                          static_cast<uint64_t>(d.M), static_cast<uint64_t>(ld) * eb, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
                if (s) return s;
                p->out_ptr[i] = dst[i];
            }
            p->out_n = n_dst; p->out_ld = ld * 1000003 + col_offset;
        }
    } else if (p->out_n == 0) {
        p->out.m[0] = p->tm_a;                  // a valid descriptor the kernel never stores through
    }
    // the split tail: only with one destination (its units finish their tiles with plain stores to C); several
    // destinations run whole tiles
    const bool tail = p->tail_tiles > 0 && n_dst == 1;
    if (p->tail_tiles > 0 && !tail) {
        const int tiles = cp.tail_first + p->tail_tiles;
        cp.tail_first = tiles; cp.tail_split = 1; cp.total_units = tiles;
    }
    if (tail) cp.tail_target = ++p->tail_seq * static_cast<uint32_t>(p->cc.epi_warps * p->tail_split);
    cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[1];
    launch_config_cluster(p, cfg, attr, stream);
    void* cargs[4] = {&p->tm_a, &p->tm_b, &p->out, &cp};
    BLZ_CUDA(cudaLaunchKernelExC(&cfg, p->cc.fn, cargs));
    return BLZ_OK;
}

}  // namespace

extern "C" {

int blz_version(void) { return 3; }

const char* blz_status_string(blz_status s) {
    switch (s) {
        case BLZ_OK: return "ok";
        case BLZ_ERR_INVALID_ARGUMENT: return "invalid argument";
        case BLZ_ERR_UNSUPPORTED: return "unsupported combination";
        case BLZ_ERR_CUDA: return "CUDA call failed";
        case BLZ_ERR_DEVICE_TIMEOUT: return "device-side wait ran out";
        case BLZ_ERR_NO_DEVICE: return "no sm_100 device";
        case BLZ_ERR_TOO_LARGE: return "size exceeds the stated maximum";
        case BLZ_ERR_OUT_OF_MEMORY: return "out of device memory";
    }
    return "unknown status";
}

int blz_last_cuda_error(void) { return g_last_cuda_error; }
const char* blz_last_cuda_error_string(void) { return g_last_cuda_error_text; }

int64_t blz_tiled_scales_bytes(int64_t rows, int64_t K) {
    if (rows <= 0 || K <= 0) return 0;
    return sf_row_blocks(rows) * sf_katoms(K) * 512;
}

blz_status blz_gemm_plan_create(const blz_gemm_desc* desc, blz_gemm_plan** out_plan) {
    if (!out_plan) return BLZ_ERR_INVALID_ARGUMENT;
    *out_plan = nullptr;
    blz_status s = validate(desc);
    if (s) return s;
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return BLZ_ERR_NO_DEVICE;
    cudaDeviceProp prop;
    if (!cuda_ok(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties")) return BLZ_ERR_NO_DEVICE;
    if (prop.major != 10) return BLZ_ERR_NO_DEVICE;

    blz_gemm_plan* p = new (std::nothrow) blz_gemm_plan();
    if (!p) return BLZ_ERR_OUT_OF_MEMORY;
    p->desc = *desc;
    if (p->desc.a_scale == 0.0f) p->desc.a_scale = 1.0f;
    if (p->desc.b_scale == 0.0f) p->desc.b_scale = 1.0f;
    p->device = dev;
    p->num_sms = prop.multiProcessorCount;
    p->variant = desc->variant;
    switch (desc->kind) {
        case BLZ_GEMM_F16: case BLZ_GEMM_BF16: case BLZ_GEMM_W4A16_F16: case BLZ_GEMM_W4A16_BF16: p->mma_kind = MMA_F16; break;
        case BLZ_GEMM_FP8: p->mma_kind = MMA_F8; break;
        default: p->mma_kind = MMA_NVF4; break;
    }
    const bool w4a16 = desc->kind == BLZ_GEMM_W4A16_F16 || desc->kind == BLZ_GEMM_W4A16_BF16;

    auto fail = [&](blz_status st) { blz_gemm_plan_destroy(p); return st; };

    void* st_mem = nullptr;
    if ((s = dev_alloc(p, &st_mem, sizeof(int), true))) return fail(s);
    p->status = static_cast<int*>(st_mem);
    p->a_used = desc->A;
    if ((s = prepare_b(p))) return fail(s);
    if ((s = prepare_a_scales(p))) return fail(s);

    // Skinny activations stream the weights once through the decode kernels (every kind).  Up to 64
    // rows automatically; W4A16 up to 128 (its alternative is a 16-bit copy of the weights per call).
    // The 128-row forms of the FP8 and 16-bit kernels exist (explicit variant) but lose to the tiled
    // kernel: both re-read the activations once per 128 weight rows and are bound by L2 -> SM traffic.
    const int decode_max_m = desc->kind == BLZ_GEMM_NVFP4 ? 64 : 128;
    // ... unless the tiled kernel would split K four ways (few tiles, long K): measured 27 against 42 us
    // for 128 x 4096 x 11008
    const bool w4_tiled_split = w4a16 && desc->M > 64 && ceil_div(desc->N, 128) * 4 <= p->num_sms && desc->K >= 8192 && desc->epilogue != BLZ_EPI_SWIGLU;
    const int decode_auto_m = (w4a16 && !w4_tiled_split) ? 128 : 64;
    const bool want_decode = desc->variant == BLZ_VARIANT_DECODE || (desc->variant == BLZ_VARIANT_AUTO && desc->M <= decode_auto_m);
    // M > 128: the tiled kernel expands the packed weights stage by stage in shared memory (no 16-bit copy, one
    // launch; every CTA re-expands the tiles it uses, which costs 8 % at 4096 x 22016 x 4096: 1427 against 1556
    // TFLOP/s).  Callers whose weights are static ask for a plan-owned 16-bit copy made once
    // (BLZ_FLAG_STATIC_WEIGHTS).  BLZ_W4A16_PREPASS=1 forces the copy to be re-made by every execute (tuning).
    const bool prepass = env_int("BLZ_W4A16_PREPASS", 0) != 0;
    const bool static_w = w4a16 && !want_decode && (desc->flags & BLZ_FLAG_STATIC_WEIGHTS) != 0;
    if (w4a16 && !want_decode && (prepass || static_w || desc->variant == BLZ_VARIANT_QUAD_512x256)) {
        // The tiled kernels consume 16-bit weights: the packed weights are expanded into this buffer
        // (q * block scale, exact in 16 bits; the fp32 tensor scale goes into alpha) -- by every execute,
        // or once, here, when the caller declared them static.
        if ((s = dev_alloc(p, &p->own_w16, static_cast<int64_t>(desc->N) * desc->K * 2, false))) return fail(s);
        p->w16_static = static_w;
        p->launches = static_w ? 1 : 2;
        if (static_w && (s = expand_weights(p, nullptr))) return fail(s);
    }

    if (want_decode) {
        if (desc->M > decode_max_m) return fail(BLZ_ERR_UNSUPPORTED);
        p->variant = BLZ_VARIANT_DECODE;
        if ((s = decode_setup(p))) return fail(s);
    } else {
        const void* b_tc = (w4a16 && p->own_w16) ? p->own_w16 : p->b_used;
        const void* keep = p->b_used;
        p->b_used = b_tc;
        int v = desc->variant;
        if (v == BLZ_VARIANT_AUTO) v = choose_tile_variant(p, w4a16 && p->own_w16 == nullptr);
        if (v == BLZ_VARIANT_PAIR_256x384) s = setup_cluster(p, 2, 1, true);
        else if (v == BLZ_VARIANT_QUAD_512x256) s = setup_cluster(p, 2, 2);
        else if (v == BLZ_VARIANT_PAIR_256x256) s = setup_cluster(p, 2);
        else if (v == BLZ_VARIANT_PAIR_256x128) s = setup_cluster(p, 2, 1, false, true);
        else if (v == BLZ_VARIANT_TILE_128x128) s = setup_cluster(p, 1);
        else s = BLZ_ERR_INVALID_ARGUMENT;
        p->b_used = keep;
        if (s) return fail(s);
    }
    if (!cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize")) return fail(BLZ_ERR_CUDA);
    *out_plan = p;
    return BLZ_OK;
}

blz_status blz_gemm_execute(blz_gemm_plan* p, void* C, void* stream_v) {
    if (!p || !C) return BLZ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const blz_gemm_desc& d = p->desc;
    if (p->variant == BLZ_VARIANT_DECODE) return decode_launch(p, C, stream);

    void* one[1] = {C};
    return launch_cluster(p, 1, one, d.ldc ? d.ldc : (d.epilogue == BLZ_EPI_SWIGLU ? d.N / 2 : d.N), 0, stream);
}

blz_status blz_gemm_execute_gather(blz_gemm_plan* p, int32_t n_dst, void* const* dst, int64_t ld_total, int64_t col_offset, void* stream_v) {
    if (!p || !dst || n_dst < 1 || n_dst > BLZ_MAX_DST) return BLZ_ERR_INVALID_ARGUMENT;
    if (p->variant == BLZ_VARIANT_DECODE) return BLZ_ERR_UNSUPPORTED;
    const blz_gemm_desc& d = p->desc;
    if (ld_total < col_offset + d.N || col_offset < 0) return BLZ_ERR_INVALID_ARGUMENT;
    if (d.epilogue == BLZ_EPI_RESIDUAL_ADD || d.epilogue == BLZ_EPI_SWIGLU || p->split_k > 1) return BLZ_ERR_UNSUPPORTED;
    for (int i = 0; i < n_dst; ++i) if (!dst[i]) return BLZ_ERR_INVALID_ARGUMENT;
    return launch_cluster(p, n_dst, dst, ld_total, col_offset, static_cast<cudaStream_t>(stream_v));
}

blz_status blz_gemm_plan_set_a(blz_gemm_plan* p, const void* A, const void* A_sf, float a_scale) {
    if (!p || !A) return BLZ_ERR_INVALID_ARGUMENT;
    blz_gemm_desc& d = p->desc;
    if (d.kind == BLZ_GEMM_NVFP4) {
        if (!A_sf || d.a_sf_layout != BLZ_SF_TILED) return BLZ_ERR_INVALID_ARGUMENT;
        d.A_sf = A_sf;
        p->sfa_used = static_cast<const uint8_t*>(A_sf);
    }
    d.A = A;
    p->a_used = A;
    if (a_scale != 0.0f) d.a_scale = a_scale;
    if (p->variant == BLZ_VARIANT_DECODE) return decode_rebind_a(p);
    p->cp.sfa = p->sfa_used;
    const int64_t rb = row_bytes(p->mma_kind, d.K);
    return encode_map(&p->tm_a, A, static_cast<uint64_t>(rb), static_cast<uint64_t>(d.M), static_cast<uint64_t>(rb), 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
}

blz_status blz_gemm_plan_check(blz_gemm_plan* p, void* stream_v) {
    if (!p) return BLZ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    BLZ_CUDA(cudaStreamSynchronize(stream));
    int word = 0;
    BLZ_CUDA(cudaMemcpy(&word, p->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (word != 0) {
        g_last_cuda_error = word;
        snprintf(g_last_cuda_error_text, sizeof(g_last_cuda_error_text), "device error word 0x%x", word);
        BLZ_CUDA(cudaMemset(p->status, 0, sizeof(int)));
        if (p->tail_flags) {      // a launch that gave up may have left the units' arrival counters short: start them over
            BLZ_CUDA(cudaMemset(p->tail_flags, 0, static_cast<size_t>(p->tail_tiles) * p->cc.cg * p->cc.share * sizeof(uint32_t)));
            p->tail_seq = 0;
        }
        return BLZ_ERR_DEVICE_TIMEOUT;
    }
    return BLZ_OK;
}

blz_status blz_gemm_plan_info(const blz_gemm_plan* p, blz_plan_info* info) {
    if (!p || !info) return BLZ_ERR_INVALID_ARGUMENT;
    memset(info, 0, sizeof(*info));
    info->variant = p->variant;
    if (p->variant == BLZ_VARIANT_DECODE) {
        info->tile_m = p->decode_mma_n; info->tile_n = 128;
        info->stages = p->decode_stages; info->split_k = p->decode_split;
        info->grid = p->grid; info->smem_bytes = p->decode_smem; info->tmem_cols = p->decode_tmem;
    } else {
        info->tile_m = 128 * p->cc.cg * p->cc.share; info->tile_n = p->cc.bn;
        info->stages = p->cc.stages; info->split_k = p->split_k;
        info->grid = p->grid; info->smem_bytes = p->cc.smem; info->tmem_cols = p->cc.tmem_cols;
    }
    info->launches = p->launches;
    info->scheduler = p->clc ? 1 : 0;
    info->tail_tiles = p->tail_tiles; info->tail_split = p->tail_tiles ? p->tail_split : 1;
    info->workspace_bytes = p->owned_bytes;
    return BLZ_OK;
}

blz_status blz_gemm_plan_refresh_weights(blz_gemm_plan* p, void* stream_v) {
    if (!p) return BLZ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    blz_status s = convert_b(p, stream);                     // plan-owned K-major / tiled copies, where the plan made any
    if (s) return s;
    if (!p->own_w16 || !p->w16_static) return BLZ_OK;
    return expand_weights(p, stream);
}

blz_status blz_gemm_plan_destroy(blz_gemm_plan* p) {
    if (!p) return BLZ_OK;
    cudaFree(p->own_b); cudaFree(p->own_sfa); cudaFree(p->own_sfb); cudaFree(p->own_w16); cudaFree(p->own_partial); cudaFree(p->own_tail); cudaFree(p->tail_flags);
    cudaFree(p->status);
    (void)cudaGetLastError();
    delete p;
    return BLZ_OK;
}

blz_status blz_gemm_launch(const blz_gemm_desc* desc, void* C, void* stream) {
    blz_gemm_plan* p = nullptr;
    blz_status s = blz_gemm_plan_create(desc, &p);
    if (s) return s;
    s = blz_gemm_execute(p, C, stream);
    if (s == BLZ_OK) s = blz_gemm_plan_check(p, stream);
    blz_gemm_plan_destroy(p);
    return s;
}

// ------------------------------------------------------------ bounded-wait self test

}  // extern "C"

namespace {
// One CTA waits on a barrier nobody will ever arrive on, with the same bounded wait every kernel of
// this library uses, gives up after `limit_ns`, records the error word and returns normally.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int* status, unsigned long long* waited_ns) {
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ int abort_flag;
    const uint32_t bar = smem_u32(&bar_storage);
    if (threadIdx.x == 0) { mbar_init(bar, 1); abort_flag = 0; fence_mbar_init(); }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint64_t t0 = global_timer_ns();
        const bool ok = mbar_wait_limit(bar, 0u, &abort_flag, limit_ns);
        if (waited_ns) *waited_ns = global_timer_ns() - t0;
        if (!ok) atomicCAS(status, 0, BLZ_DEV_TIMEOUT_PRODUCER);
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_inval(bar);
}
}  // namespace

extern "C" {

blz_status blz_wait_probe(uint64_t limit_ns, int32_t* d_status, uint64_t* d_waited_ns, void* stream_v) {
    if (!d_status || limit_ns == 0 || limit_ns > 100000000ull) return BLZ_ERR_INVALID_ARGUMENT;   // at most 100 ms
    wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_v)>>>(limit_ns, d_status, reinterpret_cast<unsigned long long*>(d_waited_ns));
    BLZ_CUDA(cudaGetLastError());
    return BLZ_OK;
}

// ------------------------------------------------------------ peer-visible buffers

blz_status blz_peer_buffer_create(int64_t bytes, void** ptr, uint8_t* handle64) {
    if (!ptr || !handle64 || bytes <= 0) return BLZ_ERR_INVALID_ARGUMENT;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!cuda_ok(cudaMalloc(ptr, static_cast<size_t>(bytes)), "cudaMalloc")) return BLZ_ERR_OUT_OF_MEMORY;
    cudaIpcMemHandle_t h;
    if (!cuda_ok(cudaIpcGetMemHandle(&h, *ptr), "cudaIpcGetMemHandle")) { cudaFree(*ptr); *ptr = nullptr; return BLZ_ERR_CUDA; }
    memcpy(handle64, &h, 64);
    return BLZ_OK;
}

blz_status blz_peer_buffer_open(const uint8_t* handle64, void** ptr) {
    if (!ptr || !handle64) return BLZ_ERR_INVALID_ARGUMENT;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    BLZ_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return BLZ_OK;
}

blz_status blz_peer_buffer_close(void* ptr) {
    if (!ptr) return BLZ_OK;
    BLZ_CUDA(cudaIpcCloseMemHandle(ptr));
    return BLZ_OK;
}

blz_status blz_peer_buffer_destroy(void* ptr) {
    if (!ptr) return BLZ_OK;
    BLZ_CUDA(cudaFree(ptr));
    return BLZ_OK;
}

// ------------------------------------------------------------ preparation

blz_status blz_amax(const void* x, int32_t x_dtype, int64_t n, float* d_amax, void* stream_v) {
    if (!x || !d_amax || n <= 0) return BLZ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int g = grid_for(n, 256 * 8);
    if (x_dtype == BLZ_F32) amax_kernel<float><<<g, 256, 0, stream>>>(static_cast<const float*>(x), n, d_amax);
    else if (x_dtype == BLZ_F16) amax_kernel<__half><<<g, 256, 0, stream>>>(static_cast<const __half*>(x), n, d_amax);
    else if (x_dtype == BLZ_BF16) amax_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), n, d_amax);
    else return BLZ_ERR_INVALID_ARGUMENT;
    BLZ_CUDA(cudaGetLastError());
    return BLZ_OK;
}

blz_status blz_quantize_fp8(const void* x, int32_t x_dtype, int64_t n, const float* d_amax, uint8_t* q, float* d_scales, void* stream_v) {
    if (!x || !d_amax || !q || n <= 0) return BLZ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int g = grid_for(n, 256 * 4);
    if (x_dtype == BLZ_F32) quantize_fp8_kernel<float><<<g, 256, 0, stream>>>(static_cast<const float*>(x), n, d_amax, q, d_scales);
    else if (x_dtype == BLZ_F16) quantize_fp8_kernel<__half><<<g, 256, 0, stream>>>(static_cast<const __half*>(x), n, d_amax, q, d_scales);
    else if (x_dtype == BLZ_BF16) quantize_fp8_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), n, d_amax, q, d_scales);
    else return BLZ_ERR_INVALID_ARGUMENT;
    BLZ_CUDA(cudaGetLastError());
    return BLZ_OK;
}

blz_status blz_quantize_nvfp4(const void* x, int32_t x_dtype, int64_t rows, int64_t K, const float* d_amax, uint8_t* data, uint8_t* sf,
                              int32_t sf_layout, float* d_global, void* stream_v) {
    if (!x || !d_amax || !data || !sf || rows <= 0 || K <= 0 || (K % 16) != 0) return BLZ_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(data) & 7u) != 0) return BLZ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int tiled = sf_layout == BLZ_SF_TILED ? 1 : 0;
    if (tiled) BLZ_CUDA(cudaMemsetAsync(sf, 0, static_cast<size_t>(blz_tiled_scales_bytes(rows, K)), stream));
    const int g = grid_for(rows * (K / 16), 256);
    const long long ka = sf_katoms(K);
    if (x_dtype == BLZ_F32) quantize_nvfp4_kernel<float><<<g, 256, 0, stream>>>(static_cast<const float*>(x), rows, K, d_amax, data, sf, tiled, ka, d_global);
    else if (x_dtype == BLZ_F16) quantize_nvfp4_kernel<__half><<<g, 256, 0, stream>>>(static_cast<const __half*>(x), rows, K, d_amax, data, sf, tiled, ka, d_global);
    else if (x_dtype == BLZ_BF16) quantize_nvfp4_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), rows, K, d_amax, data, sf, tiled, ka, d_global);
    else return BLZ_ERR_INVALID_ARGUMENT;
    BLZ_CUDA(cudaGetLastError());
    return BLZ_OK;
}

blz_status blz_tile_scales(const uint8_t* sf, int64_t rows, int64_t K, int64_t row_stride, int64_t blk_stride, uint8_t* tiled, void* stream_v) {
    if (!sf || !tiled || rows <= 0 || K <= 0 || (K % 16) != 0) return BLZ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    BLZ_CUDA(cudaMemsetAsync(tiled, 0, static_cast<size_t>(blz_tiled_scales_bytes(rows, K)), stream));
    const int64_t kb = K / 16;
    tile_scales_kernel<<<grid_for(rows * kb, 256), 256, 0, stream>>>(sf, rows, kb, row_stride, blk_stride, sf_katoms(K), tiled);
    BLZ_CUDA(cudaGetLastError());
    return BLZ_OK;
}

blz_status blz_interleave_gate_up(const void* gate, const void* up, void* out, int64_t n_groups, int64_t group_bytes, void* stream_v) {
    if (!gate || !up || !out || n_groups <= 0 || group_bytes <= 0 || (group_bytes % 4) != 0) return BLZ_ERR_INVALID_ARGUMENT;
    if (((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) & 3u) != 0) return BLZ_ERR_INVALID_ARGUMENT;
    const int64_t words = group_bytes / 4;
    interleave_groups_kernel<<<grid_for(n_groups * words, 256), 256, 0, static_cast<cudaStream_t>(stream_v)>>>(
        static_cast<const uint32_t*>(gate), static_cast<const uint32_t*>(up), static_cast<uint32_t*>(out), n_groups, words);
    BLZ_CUDA(cudaGetLastError());
    return BLZ_OK;
}

}  // extern "C"
