// decode_static.cu -- blz_gemm_nvfp4_decode_static: the skinny-M NVFP4 GEMM for callers that must
// not allocate device memory.
//
// Who that is: serving runtimes that hand every byte of HBM to their own arena when they start
// (weights, KV cache, activation pools) and then forbid cudaMalloc for the rest of the process --
// a late allocation there either fails or forces the arena to shrink -- and latency-critical loops
// in which an allocation's implicit device synchronisation is not acceptable.  Plans own their
// device memory through cudaMalloc (status word, repacked operands, the tiled kernel's split-K
// partial sums); this entry point keeps its split-K workspace in a fixed array that is part of the
// library image instead.
//
// The kernel is decode_nvf4_kernel (decode_kernel.cuh): K splits write fp32 partial sums to global
// memory and the CTA that arrives last at a tile (an atomic ticket) adds them in split order.  It
// is NOT the kernel a plan with BLZ_VARIANT_DECODE runs (decode_stream_kernel reduces its splits
// through distributed shared memory and needs no scratch); both cut K with the same rule
// (decode_split.h) and add the splits in the same order, so their results agree bit for bit.
//
// The array is part of the module image: the driver places it in device memory when the module is
// loaded, which with lazy module loading happens at the first call on a device (the symbol lookup
// below).  A caller whose arena takes all of HBM must therefore make its first call on each
// device -- any small shape -- BEFORE it sizes the arena; later calls touch no allocator.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "../../include/blaze_b200.h"
#include "decode_kernel.cuh"
#include "decode_split.h"

using namespace blz;

namespace {

// Layout of the fixed scratch array:
//   [0, 4096)                     tile counters (1024 x int)     -- must be zero when a call starts
//   [4096, 4352)                  error word of the last call
//   [8192, 8192 + PARTIAL_BYTES)  fp32 partial sums of the K splits
constexpr size_t MAX_TILES = 1024;                        // N <= 131072
constexpr size_t PARTIAL_BYTES = 8u << 20;                // 8 MiB of partial sums
constexpr size_t COUNTER_OFF = 0, STATUS_OFF = 4096, PARTIAL_OFF = 8192;
constexpr size_t SCRATCH_BYTES = PARTIAL_OFF + PARTIAL_BYTES;

// Every GPU that loads this library holds this array until the process exits.
static __device__ __align__(256) unsigned char g_decode_scratch[SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_setup_mutex;
// Per-device state, written once under the mutex; the pointer is published last (release) and read
// with acquire, so a thread that sees it also sees the SM count.
std::atomic<unsigned char*> g_scratch_ptr[MAX_DEVICES];   // device address of g_decode_scratch, per device
int g_num_sms[MAX_DEVICES] = {};

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;

struct Choice { const void* fn; int mma_n, smem; };
template <int MMA_N, int STAGES> Choice choice() {
    return Choice{reinterpret_cast<const void*>(&decode_nvf4_kernel<MMA_N, STAGES>), MMA_N, static_cast<int>(DecodeConfig<MMA_N, STAGES>::SMEM_BYTES)};
}
Choice pick(int M) { return M <= 16 ? choice<16, 5>() : M <= 32 ? choice<32, 4>() : choice<64, 3>(); }

// Once per device, with that device current: resolve the device address of the scratch array
// (in host code the array's name is only a handle for the runtime, never a device pointer), raise
// the kernels' dynamic shared-memory limit and look up the tensor-map encoder.
blz_status setup_device(int dev) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev].load(std::memory_order_acquire)) return BLZ_OK;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) { (void)cudaGetLastError(); return BLZ_ERR_NO_DEVICE; }
    if (prop.major != 10) return BLZ_ERR_NO_DEVICE;
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
    // loading the module places the array in device memory: the one implicit allocation of this entry point
    if (e == cudaErrorMemoryAllocation) { (void)cudaGetLastError(); return BLZ_ERR_OUT_OF_MEMORY; }
    if (e != cudaSuccess || ptr == nullptr) { (void)cudaGetLastError(); return BLZ_ERR_CUDA; }
    for (int m : {16, 32, 64}) {
        const Choice c = pick(m);
        e = cudaFuncSetAttribute(c.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, c.smem);
        if (e != cudaSuccess) { (void)cudaGetLastError(); return e == cudaErrorMemoryAllocation ? BLZ_ERR_OUT_OF_MEMORY : BLZ_ERR_CUDA; }
    }
    if (!g_encode) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            return BLZ_ERR_CUDA;
        }
        g_encode = reinterpret_cast<EncodeFn>(f);
    }
    g_num_sms[dev] = prop.multiProcessorCount;
    g_scratch_ptr[dev].store(static_cast<unsigned char*>(ptr), std::memory_order_release);
    return BLZ_OK;
}

// byte-typed 2-D map: rows of `row_bytes`, box 128 bytes x box_rows, 128-byte swizzle
bool encode_rows(CUtensorMap* m, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows) {
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" blz_status blz_gemm_nvfp4_decode_static(const void* A, const void* A_sf_tiled, float a_scale, const void* B, const void* B_sf_tiled,
                                                   float b_scale, int32_t M, int32_t N, int32_t K, void* C, int32_t out_dtype, int64_t ldc,
                                                   int32_t* d_status, void* stream_v) {
    if (!A || !A_sf_tiled || !B || !B_sf_tiled || !C) return BLZ_ERR_INVALID_ARGUMENT;
    if (M <= 0 || N <= 0 || K <= 0 || (K % 32) != 0) return BLZ_ERR_INVALID_ARGUMENT;
    if (out_dtype < BLZ_F16 || out_dtype > BLZ_F32 || (ldc != 0 && ldc < N)) return BLZ_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u) || (reinterpret_cast<uintptr_t>(A_sf_tiled) & 15u) ||
        (reinterpret_cast<uintptr_t>(B_sf_tiled) & 15u))
        return BLZ_ERR_INVALID_ARGUMENT;
    if (M > 64) return BLZ_ERR_TOO_LARGE;                           // the skinny kernel holds at most 64 activation rows
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return BLZ_ERR_NO_DEVICE; }
    if (dev < 0 || dev >= MAX_DEVICES) return BLZ_ERR_UNSUPPORTED;
    unsigned char* scratch = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!scratch) {
        blz_status s = setup_device(dev);
        if (s) return s;
        scratch = g_scratch_ptr[dev].load(std::memory_order_acquire);
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    const Choice kc = pick(M);
    DecodeKernelParams dp = {};
    dp.M = M; dp.N = N;
    dp.n_tiles = (N + 127) / 128;
    const int64_t row_bytes = K / 2;
    dp.k_stages_total = static_cast<int>((row_bytes + 127) / 128);
    // the same K partition as the plan path (same rule, same BLZ_DECODE_SPLIT override), so both give bit-identical sums
    dp.split = decode_pick_split(dp.n_tiles, dp.k_stages_total, g_num_sms[dev], decode_max_split(kc.mma_n), decode_split_override());
    dp.stages_per_split = (dp.k_stages_total + dp.split - 1) / dp.split;
    if (static_cast<size_t>(dp.n_tiles) > MAX_TILES) return BLZ_ERR_TOO_LARGE;
    const size_t partial_need = dp.split > 1 ? static_cast<size_t>(dp.split) * kc.mma_n * dp.n_tiles * 128 * sizeof(float) : 0;
    if (partial_need > PARTIAL_BYTES) return BLZ_ERR_TOO_LARGE;

    CUtensorMap tm_w, tm_x;
    if (!encode_rows(&tm_w, B, static_cast<uint64_t>(row_bytes), static_cast<uint64_t>(N), 128)) return BLZ_ERR_CUDA;
    if (!encode_rows(&tm_x, A, static_cast<uint64_t>(row_bytes), static_cast<uint64_t>(M), static_cast<uint32_t>(kc.mma_n))) return BLZ_ERR_CUDA;

    dp.idesc = make_idesc_nvf4(128, static_cast<uint32_t>(kc.mma_n));
    dp.sfw = static_cast<const uint8_t*>(B_sf_tiled);
    dp.sfx = static_cast<const uint8_t*>(A_sf_tiled);
    int64_t katoms = (static_cast<int64_t>(K) + 63) / 64;
    katoms = (katoms + 3) / 4 * 4;
    dp.sf_katoms = static_cast<int>(katoms);
    dp.partial = reinterpret_cast<float*>(scratch + PARTIAL_OFF);
    dp.counters = reinterpret_cast<int*>(scratch + COUNTER_OFF);
    // Without a status word from the caller a give-up on a bounded wait is NOT reported: the word then
    // lands in the shared array, where the next call clears it.
    dp.status = d_status ? d_status : reinterpret_cast<int*>(scratch + STATUS_OFF);
    EpilogueParams& e = dp.epi;
    e.C = C; e.bias = nullptr; e.residual = nullptr;
    e.ldc = ldc ? ldc : N; e.ldr = e.ldc;
    e.alpha = (a_scale == 0.0f ? 1.0f : a_scale) * (b_scale == 0.0f ? 1.0f : b_scale);
    e.mode = EPI_NONE; e.out_type = out_dtype; e.vec_ok = 0;

    // The array keeps whatever the previous call left behind: the counters (and the fallback error
    // word) have to start at zero; partial sums are always written before they are read.
    if (cudaMemsetAsync(scratch, 0, STATUS_OFF + 256, stream) != cudaSuccess) { (void)cudaGetLastError(); return BLZ_ERR_CUDA; }
    void* args[3] = {&tm_w, &tm_x, &dp};
    if (cudaLaunchKernel(kc.fn, dim3(static_cast<unsigned>(dp.n_tiles * dp.split)), dim3(256), args, static_cast<size_t>(kc.smem), stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return BLZ_ERR_CUDA;
    }
    return BLZ_OK;
}
