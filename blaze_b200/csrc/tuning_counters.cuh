// tuning_counters.cuh -- included only by tuning builds (-DBLZ_KERNEL_TIMING; `python -m blaze_b200.tuning`
// makes one beside the shipped library).  Per-role cycle accounting and an event trace of CTA 0, read back
// through two extra entry points that the shipped library does not have.
//
// Counter slots per CTA (16 x u64), tiled kernel: 0 producer wait-empty, 1 producer total, 2 MMA wait for a
// loaded stage, 3 MMA wait for the accumulator, 4 MMA total, 5 epilogue wait-full, 6 epilogue work, 7 epilogue
// total, 8 tiles; a K-split unit of the tail (first epilogue warp): 9 accumulator -> scratch, 10 fence and publish,
// 11 wait for the tile's other units, 12 sum / finish / store.  The skinny-M kernels use the slots as stamps along their dependent chain (see the kernels).
#pragma once

namespace blz {

__device__ unsigned long long g_blz_timing[1024 * 16];
// event trace of CTA 0: region r (0 = MMA thread, one stamp per stage; 1 = accumulator free seen by the MMA thread;
// 2, 3 = epilogue events), entry i
__device__ unsigned long long g_blz_trace[4 * 4096];

}  // namespace blz

#define BLZ_T_DECL(name) long long name = 0
#define BLZ_T_NOW() clock64()
#define BLZ_T_ADD(acc, t0) acc += clock64() - (t0)
#define BLZ_T_STORE(slot, v) blz::g_blz_timing[(blockIdx.x & 1023) * 16 + (slot)] = static_cast<unsigned long long>(v)
#define BLZ_T_STORE_IF(cond, slot, v) do { if (cond) BLZ_T_STORE(slot, v); } while (0)
#define BLZ_TRACE(region, i) do { if (blockIdx.x == 0 && (i) < 4096) blz::g_blz_trace[(region) * 4096 + (i)] = clock64(); } while (0)

#ifdef BLZ_TUNING_ENTRY_POINTS
extern "C" int blz_debug_read_timing(unsigned long long* out, int n_words) {
    if (cudaDeviceSynchronize() != cudaSuccess) return 3;
    return cudaMemcpyFromSymbol(out, blz::g_blz_timing, sizeof(unsigned long long) * static_cast<size_t>(n_words)) == cudaSuccess ? 0 : 3;
}
extern "C" int blz_debug_read_trace(unsigned long long* out, int n_words) {
    if (cudaDeviceSynchronize() != cudaSuccess) return 3;
    return cudaMemcpyFromSymbol(out, blz::g_blz_trace, sizeof(unsigned long long) * static_cast<size_t>(n_words)) == cudaSuccess ? 0 : 3;
}
#endif
