// gemm/tmem_utils.cuh -- Blaze's low-level tensor-memory / tcgen05 helper names
// (include/gemm/tmem_utils.cuh:22-589 there; used by tests/test_sm100_primitives.cu), written
// against the PTX ISA directly.  Same names and argument meaning; device code only.
//
// Differences: tensor-memory reads address the calling warp's own 32 lanes explicitly
// (lane field = 32 * (warp % 4)), as the ISA requires, instead of leaving the lane field zero.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace blaze {

using tmem_addr_t = uint32_t;

// Padding (in floats) of a shared-memory row that receives accumulator rows, against bank conflicts.
constexpr int SMEM_C_PAD = 4;

// Instruction descriptor of tcgen05.mma.kind::f8f6f4: fp32 accumulate, both operands K-major.
// Formats: 0 = E4M3, 1 = E5M2, 3 = E2M3, 4 = E3M2, 5 = E2M1.  (Blaze: tmem_utils.cuh:419-433)
__device__ __host__ __forceinline__ uint32_t make_idesc_f8f6f4(uint32_t a_format, uint32_t b_format, uint32_t tile_m, uint32_t tile_n) {
    return (1u << 4) | ((a_format & 7u) << 7) | ((b_format & 7u) << 10) | (((tile_n >> 3) & 0x3Fu) << 17) | (((tile_m >> 4) & 0x1Fu) << 24);
}

// Instruction descriptor of the block-scaled kinds: scale-factor ids in bits [4,6) (B) and
// [29,31) (A), scale format in bit 23 (0 = E4M3 scales).  (Blaze: tmem_utils.cuh:512-531)
__device__ __host__ __forceinline__ uint32_t make_idesc_blkscaled(uint32_t a_format, uint32_t b_format, uint32_t tile_m, uint32_t tile_n,
                                                                  uint32_t sfa_id, uint32_t sfb_id, uint32_t scale_format = 0) {
    return ((sfb_id & 3u) << 4) | ((a_format & 7u) << 7) | ((b_format & 7u) << 10) | (((tile_n >> 3) & 0x3Fu) << 17) |
           ((scale_format & 1u) << 23) | (((tile_m >> 4) & 0x1Fu) << 24) | ((sfa_id & 3u) << 29);
}

#ifdef __CUDACC__

// ---- allocation: executed by one whole warp; the base address lands in shared memory
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_tmem_addr, uint32_t num_columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_tmem_addr))), "r"(num_columns) : "memory");
}
__device__ __forceinline__ void tmem_alloc_cta2(uint32_t* smem_tmem_addr, uint32_t num_columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_tmem_addr))), "r"(num_columns) : "memory");
}
__device__ __forceinline__ void tmem_dealloc(tmem_addr_t addr, uint32_t num_columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(num_columns) : "memory");
}
__device__ __forceinline__ void tmem_dealloc_cta2(tmem_addr_t addr, uint32_t num_columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(num_columns) : "memory");
}

// ---- reads: lane i of the warp receives 8 consecutive columns of row 32 * (warp % 4) + i
__device__ __forceinline__ void tmem_load_8xf32(float out[8], tmem_addr_t taddr, int col) {
    const uint32_t addr = taddr + (static_cast<uint32_t>((threadIdx.x >> 5) & 3u) << 21) + static_cast<uint32_t>(col);   // lane field: 32 * quarter << 16
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=f"(out[0]), "=f"(out[1]), "=f"(out[2]), "=f"(out[3]), "=f"(out[4]), "=f"(out[5]), "=f"(out[6]), "=f"(out[7])
                 : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Accumulator rows -> shared memory [128][smem_stride] floats; every warp copies its own 32 rows.
__device__ __forceinline__ void tmem_store_to_smem_warp(float* smem_out, tmem_addr_t taddr, int tile_n, int smem_stride, int warp_id) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = warp_id * 32 + static_cast<int>(threadIdx.x & 31u);
    for (int c0 = 0; c0 < tile_n; c0 += 8) {
        float v[8];
        tmem_load_8xf32(v, taddr, c0);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 8; ++c) smem_out[row * smem_stride + c0 + c] = v[c];
    }
}
__device__ __forceinline__ void tmem_store_to_smem_warp(float* smem_out, tmem_addr_t taddr, int tile_n, int warp_id) {
    tmem_store_to_smem_warp(smem_out, taddr, tile_n, tile_n, warp_id);
}
__device__ __forceinline__ void tmem_store_to_smem(float* smem_out, tmem_addr_t taddr, int tile_n) {
    tmem_store_to_smem_warp(smem_out, taddr, tile_n, tile_n, static_cast<int>(threadIdx.x >> 5));
}

// ---- shared-memory operand descriptor: address / 16 in bits [0,14), stride between 8-row groups
//      / 16 in [32,46), version 1 in [46,48), layout in [61,64): 0 none, 2 128-byte, 4 64-byte,
//      6 32-byte swizzle.  (Blaze: tmem_utils.cuh:372-381)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t stride_bytes, uint32_t layout_type) {
    return (static_cast<uint64_t>(smem_addr >> 4) & 0x3FFFull) | ((static_cast<uint64_t>(stride_bytes >> 4) & 0x3FFFull) << 32) |
           (1ull << 46) | (static_cast<uint64_t>(layout_type & 7u) << 61);
}
__device__ __forceinline__ uint64_t make_sf_smem_desc(uint32_t smem_addr, uint32_t stride_bytes) { return make_smem_desc(smem_addr, stride_bytes, 0); }

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one_sync() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// ---- block-scaled pieces
// 32 rows x 16 bytes of scale factors, replicated to the four 32-lane quarters: four columns.
__device__ __forceinline__ void tcgen05_cp_32x128b_warpx4(uint32_t tmem_col, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(smem_desc) : "memory");
}
// D (+)= (A * SFA)(B * SFB): E2M1 operands, one E4M3 scale per 16 values along K.
__device__ __forceinline__ void blkscaled_mma_mxf4nvf4(tmem_addr_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                       tmem_addr_t sfa_tmem, tmem_addr_t sfb_tmem, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}

// ---- cluster launch control (Blaze: tmem_utils.cuh:251-305 sketches these names and never calls them).
// clc_try_cancel asks the hardware to cancel a cluster of this grid that has not started; the 16-byte answer lands in
// shared memory and completes 16 bytes on the mbarrier (arm it with mbarrier_expect_tx(mbar, 16) first, then
// mbarrier_wait).  The answer is opaque: it is decoded with the query instructions, not by reading bits.
__device__ __forceinline__ void clc_try_cancel(void* smem_response, uint64_t* mbar_smem, uint32_t /*cta_mask*/ = 1u) {
    asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
                 ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_response))), "r"(static_cast<uint32_t>(__cvta_generic_to_shared(mbar_smem))) : "memory");
}
struct ClcResponse { uint32_t data[4]; };
// true when a cluster was cancelled, i.e. its tile now belongs to the caller
__device__ __forceinline__ bool clc_is_valid(const ClcResponse* resp) {
    uint32_t ok;
    asm volatile("{\n\t.reg .b128 rr;\n\t.reg .pred p;\n\tld.shared.b128 rr, [%1];\n\t"
                 "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, rr;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(resp))) : "memory");
    return ok != 0;
}
// x index of the cancelled cluster's first CTA (the linear tile id of a one-dimensional grid); only after clc_is_valid
__device__ __forceinline__ uint32_t clc_get_linear_id(const ClcResponse* resp) {
    uint32_t x;
    asm volatile("{\n\t.reg .b128 rr;\n\tld.shared.b128 rr, [%1];\n\t"
                 "clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %0, rr;\n\t}"
                 : "=r"(x) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(resp))) : "memory");
    return x;
}

#endif  // __CUDACC__

}  // namespace blaze
