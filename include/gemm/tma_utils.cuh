// gemm/tma_utils.cuh -- Blaze's low-level TMA / mbarrier helper names on top of this library's
// conventions, so that code written against Blaze's bring-up helpers
// (include/gemm/tma_utils.cuh:32-273 there; used by tests/test_sm100_primitives.cu) compiles here.
//
// Same names and argument meaning.  Differences, all deliberate:
//   - the tensor-map encoder is looked up through the CUDA runtime (no link against libcuda);
//   - a failed encode prints and returns with the descriptor zeroed instead of exiting;
//   - mbarrier_wait gives up after one second instead of spinning forever (it then returns; the
//     caller's data is not ready, its results will be wrong, the GPU stays usable).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>

namespace blaze {

constexpr int TMA_DESC_SIZE = 128;

struct TmaDescriptor {
    alignas(64) char data[TMA_DESC_SIZE];
};

enum class TmaSwizzle : uint32_t { NONE = 0, B32 = 1, B64 = 2, B128 = 3 };

// Row-major [rows, cols] matrix, tile of box_rows x box_cols elements (Blaze: tma_utils.cuh:62-139).
inline void create_tma_desc_2d(TmaDescriptor* desc, const void* global_ptr, CUtensorMapDataType format, uint64_t rows, uint64_t cols,
                               uint32_t box_rows, uint32_t box_cols, TmaSwizzle swizzle = TmaSwizzle::B128) {
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    std::memset(desc, 0, sizeof(*desc));
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            std::fprintf(stderr, "blaze: tensor-map encoder not available\n");
            return;
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const uint64_t elem = (format == CU_TENSOR_MAP_DATA_TYPE_UINT8) ? 1 : (format == CU_TENSOR_MAP_DATA_TYPE_FLOAT32) ? 4 : 2;
    const bool is_float = format == CU_TENSOR_MAP_DATA_TYPE_FLOAT16 || format == CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 ||
                          format == CU_TENSOR_MAP_DATA_TYPE_FLOAT32 || format == CU_TENSOR_MAP_DATA_TYPE_FLOAT64 ||
                          format == CU_TENSOR_MAP_DATA_TYPE_TFLOAT32;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * elem};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = swizzle == TmaSwizzle::B128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : swizzle == TmaSwizzle::B64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle == TmaSwizzle::B32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    const CUresult r = encode(reinterpret_cast<CUtensorMap*>(desc), format, 2, const_cast<void*>(global_ptr), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                              is_float ? CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA : CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        std::fprintf(stderr, "blaze: cuTensorMapEncodeTiled failed (%d)\n", static_cast<int>(r));
        std::memset(desc, 0, sizeof(*desc));
    }
}

__host__ __device__ constexpr uint32_t tma_tile_bytes(uint32_t box_rows, uint32_t box_cols, uint32_t elem_size) { return box_rows * box_cols * elem_size; }

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t compat_smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// coord_x walks the contiguous dimension; coord_x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_ptr, const TmaDescriptor* desc, int32_t coord_x, int32_t coord_y, uint64_t* mbar_ptr) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(compat_smem_addr(smem_ptr)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(compat_smem_addr(mbar_ptr)), "r"(coord_x), "r"(coord_y)
                 : "memory");
}

__device__ __forceinline__ void mbarrier_init(uint64_t* mbar_ptr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(compat_smem_addr(mbar_ptr)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarrier_expect_tx(uint64_t* mbar_ptr, uint32_t tx_bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(compat_smem_addr(mbar_ptr)), "r"(tx_bytes) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t* mbar_ptr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(compat_smem_addr(mbar_ptr)) : "memory");
}
__device__ __forceinline__ void mbarrier_inval(uint64_t* mbar_ptr) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(compat_smem_addr(mbar_ptr)) : "memory");
}
// Waits for the phase with parity `phase`; bounded (one second of %globaltimer).
__device__ __forceinline__ void mbarrier_wait(uint64_t* mbar_ptr, uint32_t phase) {
    const uint32_t bar = compat_smem_addr(mbar_ptr);
    uint64_t t0 = 0;
    for (uint32_t spins = 0;; ++spins) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(phase) : "memory");
        if (done) return;
        if ((spins & 255u) == 255u) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > 1000000000ull) return;
        }
    }
}

#endif  // __CUDACC__

}  // namespace blaze
