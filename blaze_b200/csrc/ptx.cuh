// ptx.cuh -- inline-PTX building blocks for sm_100a: mbarrier (bounded waits), TMA loads/stores,
// tensor-memory allocation, tcgen05 MMA / copy / load, and the descriptor encoders they need.
//
// These replace the helpers Blaze keeps in include/gemm/tma_utils.cuh (TMA + mbarrier,
// :153-261) and include/gemm/tmem_utils.cuh (TMEM alloc/ld :41-117, descriptors :372-433,
// block-scaled MMA :452-589).  Differences that matter: every wait is bounded, MMA completion is
// signalled with tcgen05.commit (never a plain arrive), and descriptor fields follow the PTX ISA
// tables for K-major 128-byte-swizzled operands.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace blz {

// How long one device-side wait may spin before the kernel gives up, records an error word and
// unwinds (frees tensor memory, returns).  Legitimate waits are microseconds.
#ifndef BLZ_WAIT_LIMIT_NS
#define BLZ_WAIT_LIMIT_NS 1000000000ull
#endif

// Error words a kernel writes to its status slot (0 = fine).
enum : int {
    BLZ_DEV_OK = 0,
    BLZ_DEV_TIMEOUT_PRODUCER = 0x101,   // waiting for a free smem stage
    BLZ_DEV_TIMEOUT_MMA_FULL = 0x102,   // waiting for a loaded smem stage
    BLZ_DEV_TIMEOUT_MMA_ACC = 0x103,    // waiting for a drained accumulator
    BLZ_DEV_TIMEOUT_EPILOGUE = 0x104,   // waiting for a finished accumulator
    BLZ_DEV_TIMEOUT_SPLITK = 0x105,
    BLZ_DEV_TIMEOUT_STORE = 0x106,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------- single-thread roles
// True in exactly one lane of a converged warp (all 32 lanes must execute it).  Roles that issue
// TMA copies and tcgen05.mma / tcgen05.commit are entered through this, not through `lane == 0`:
// those instructions take their operands from the uniform datapath, and only after elect.sync
// does the compiler keep a role's address arithmetic there.  Measured on B200 with 1024
// back-to-back 128 x 16 x 16 MMAs (A in tensor memory): 20 cycles per instruction behind
// elect.sync, 94 behind `threadIdx.x == 0`.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

#ifndef BLZ_POLL_SLEEP_NS
#define BLZ_POLL_SLEEP_NS 32
#endif

// Register budget of a warpgroup (four consecutive warps; every warp of the group must execute the same
// call).  `dec` hands registers back to the CTA's pool, `inc` takes them and waits until the pool holds
// enough -- so the new budgets of all warpgroups together must not exceed what the CTA was launched with
// (threads x registers per thread of the launch bound), or `inc` never returns.
template <int N> __device__ __forceinline__ void warpgroup_regs_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void warpgroup_regs_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// Makes freshly initialised barriers visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `cta` of this cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(bar), "r"(cta) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
#ifdef BLZ_MBAR_TEST_WAIT
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
#else
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
#endif
    return ok != 0;
}
// Bounded wait: true when the phase completed; false when `limit_ns` ran out or another role of
// this CTA already gave up (`abort_flag`, a word in shared memory, non-zero).
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, const volatile int* abort_flag, uint64_t limit_ns) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag != 0) return false;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
    return mbar_wait_limit(bar, parity, abort_flag, BLZ_WAIT_LIMIT_NS);
}
// The same bounded wait for a whole warp (all 32 lanes must call it): lane 0 polls, the others
// wait at the warp barrier without issuing shared-memory traffic.  Many warps polling one barrier
// with every lane load the shared-memory pipe that TMA completions and tcgen05.commit arrivals
// also go through.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) {
        // a failed poll backs off: sixteen pollers re-issuing mbarrier.try_wait back to back were
        // measured to delay every other barrier operation of the CTA by ~200 cycles
        const uint64_t t0 = global_timer_ns();
#pragma unroll 1
        for (int i = 0; !mbar_try_wait(bar, parity); ++i) {
            __nanosleep(BLZ_POLL_SLEEP_NS);
            if ((i & 255) == 255 && (*abort_flag != 0 || global_timer_ns() - t0 > BLZ_WAIT_LIMIT_NS)) { ok = false; break; }
        }
    }
    return __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
}
// A counter in global memory that CTAs of one grid publish to and wait on (all of them resident, and no CTA
// waits before it has published): release-add, and the bounded wait of a whole warp for the counter to reach
// `target` (wrap-safe; lane 0 polls with an acquire load, the warp barrier passes the ordering on).
__device__ __forceinline__ void red_release_gpu_add_u32(uint32_t* p, uint32_t v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool flag_wait_warp(const uint32_t* flag, uint32_t target, const volatile int* abort_flag) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) {
        const uint64_t t0 = global_timer_ns();
#pragma unroll 1
        for (int i = 0; static_cast<int32_t>(ld_acquire_gpu_u32(flag) - target) < 0; ++i) {
            __nanosleep(20);
            if ((i & 255) == 255 && (*abort_flag != 0 || global_timer_ns() - t0 > BLZ_WAIT_LIMIT_NS)) { ok = false; break; }
        }
    }
    ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
    __syncwarp();
    return ok;
}
// The same bounded wait for warps that wait long while other warps of the SM need the issue slots:
// sleeps between polls (the wake-up may come up to ~0.2 us late).
__device__ __forceinline__ bool mbar_wait_sleepy(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
    const uint64_t t0 = global_timer_ns();
#pragma unroll 1
    for (int i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(200);
        if ((i & 63) == 63) {
            if (*abort_flag != 0) return false;
            if (global_timer_ns() - t0 > BLZ_WAIT_LIMIT_NS) return false;
        }
    }
}

// ---------------------------------------------------------------------- TMA

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared, completion counted in bytes on `bar`.
// c0 is the coordinate along the contiguous dimension: c0 * element size must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* m, int c0, int c1, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(bar), "l"(policy) : "memory");
}
// CTA-pair form: the data goes to this CTA's shared memory, the completion bytes to `bar_cluster`, a
// shared::cluster address that may name a barrier of the other CTA of the pair (the leader's), so the
// pair's MMA thread sees both CTAs' tiles land on one barrier.  One source, one destination: no multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int c0, int c1, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(bar_cluster) : "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `cta` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
// arrive on a barrier given by its shared::cluster address
__device__ __forceinline__ void mbar_arrive_cluster_addr(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// Hints: bring a 2-D tile / a contiguous range into L2 without a destination (nothing to wait for).
// Same alignment rules as the loads: c0 * element size and `src` multiples of 16 bytes, `bytes` too.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(src)), "r"(bytes) : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
// Bulk copy from this CTA's shared memory into the shared memory of CTA `cta` of the cluster (same
// offsets), completion counted in bytes on that CTA's barrier.  Not a multicast: one source, one
// destination, over the SM-to-SM network instead of L2.
__device__ __forceinline__ void dsmem_copy(uint32_t dst_offset, uint32_t src, uint32_t bytes, uint32_t bar_offset, uint32_t cta) {
    asm volatile(
        "{\n\t.reg .b32 rd, rb;\n\t"
        "mapa.shared::cluster.u32 rd, %0, %4;\n\t"
        "mapa.shared::cluster.u32 rb, %3, %4;\n\t"
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [rd], [%1], %2, [rb];\n\t}"
        ::"r"(dst_offset), "r"(src), "r"(bytes), "r"(bar_offset), "r"(cta) : "memory");
}
// 2-D tiled store shared -> global (rows/columns outside the tensor are clipped by the hardware).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Orders generic-proxy writes to shared memory before async-proxy reads (TMA store, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// L2 eviction policies for TMA loads.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ------------------------------------------------------- cluster launch control
// Work stealing from the grid's own launch queue: try_cancel asks the hardware to cancel a cluster of this
// grid that has not started yet; the 16-byte answer lands in shared memory at `response` (16-byte aligned)
// and completes 16 bytes on `bar`.  One thread per cluster issues it.  If a cluster was cancelled the caller
// owns its work: clc_query returns the x index of that cluster's first CTA, otherwise -1 (nothing left to
// take).  Blaze sketches the same helpers (include/gemm/tmem_utils.cuh:273-305) and never calls them.
__device__ __forceinline__ void clc_try_cancel(uint32_t response, uint32_t bar) {
    asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
                 ::"r"(response), "r"(bar) : "memory");
}
__device__ __forceinline__ int clc_query(uint32_t response) {
    uint32_t ok, x;
    asm volatile(
        "{\n\t.reg .b128 rr;\n\t.reg .pred p;\n\t"
        "ld.shared.b128 rr, [%2];\n\t"
        "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, rr;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "mov.u32 %1, 0;\n\t"
        "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %1, rr;\n\t}"
        : "=r"(ok), "=r"(x) : "r"(response) : "memory");
    return ok ? static_cast<int>(x) : -1;
}
// cluster-scope forms for data handed between the CTAs of a cluster through shared memory: the writer
// stores with st.shared::cluster and arrives with release, the reader's wait acquires
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t addr_cluster, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr_cluster), "r"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_release_cluster_addr(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_acquire_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded, like mbar_wait
__device__ __forceinline__ bool mbar_wait_acquire_cluster(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
    const uint64_t t0 = global_timer_ns();
#pragma unroll 1
    for (int i = 0;; ++i) {
        if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
        if ((i & 127) == 127) {
            if (*abort_flag != 0) return false;
            if (global_timer_ns() - t0 > BLZ_WAIT_LIMIT_NS) return false;
        }
    }
}

// ------------------------------------------------------------ tensor memory

// Whole-warp calls.  The base address is written to shared memory at `dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// CTA-pair forms: executed by the same warp of both CTAs of the pair.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// One arrive on `bar` once every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Pair form, issued by the leader CTA: one arrive on the barrier at this offset in every CTA whose
// bit is set in `mask`, once the pair's tensor-core work issued so far has completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(mask) : "memory");
}

// 32 lanes x 32 bit, 32 / 16 consecutive columns: thread t of the warp receives row
// (32*(warp%4) + t), columns [col, col+N).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Register -> tensor memory, same addressing as the loads: thread t writes row (32*(warp%4) + t).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------- descriptors

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes wide and
// stored with the 128-byte swizzle (what a TMA box of 128 bytes x R rows with SWIZZLE_128B
// writes).  Eight rows form one 1024-byte swizzle atom, so the stride between 8-row groups is
// 1024 bytes; the leading-dimension offset is unused for this layout.  `addr` may point inside
// the first row at a multiple of 32 bytes to select one MMA-K slice; the tile base must be
// 1024-byte aligned.
__device__ __forceinline__ uint64_t make_desc_k_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);        // start address, bits [0,14)
    d |= static_cast<uint64_t>(1024u >> 4) << 32;              // stride byte offset, bits [32,46)
    d |= static_cast<uint64_t>(1) << 46;                       // descriptor version for sm_100
    d |= static_cast<uint64_t>(2) << 61;                       // layout type: 128-byte swizzle
    return d;
}
// Descriptor for a scale-factor atom: 32 rows of 16 bytes, contiguous (512 bytes), no swizzle;
// eight-row groups are 128 bytes apart.
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(128u >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}

// Instruction descriptor, kinds f16 / f8f6f4: fp32 accumulate, both operands K-major.
//   fmt (kind::f16): 0 = fp16, 1 = bf16;  fmt (kind::f8f6f4): 0 = E4M3
__host__ __device__ constexpr uint32_t make_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t mma_m, uint32_t mma_n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((mma_n >> 3) << 17) | ((mma_m >> 4) << 24);
}
// Instruction descriptor, kind mxf4nvf4 with 16-element blocks: E2M1 operands (format code 1),
// E4M3 scale factors (scale-format bit 23 = 0), scale-factor ids 0, K = 64 per instruction.
__host__ __device__ constexpr uint32_t make_idesc_nvf4(uint32_t mma_m, uint32_t mma_n) {
    return (1u << 7) | (1u << 10) | ((mma_n >> 3) << 17) | ((mma_m >> 4) << 24);
}


// ------------------------------------------------------------- narrow-format conversions
// Two E2M1 values (one byte, first value in the low nibble) -> two fp16 values.
__device__ __forceinline__ uint32_t cvt_e2m1x2_to_f16x2(uint32_t byte) {
    uint32_t r;
    asm("{\n\t.reg .b8 lo, hi;\n\t.reg .b16 h;\n\t"
        "cvt.u16.u32 h, %1;\n\t"
        "mov.b16 {lo, hi}, h;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, lo;\n\t}"
        : "=r"(r) : "r"(byte));
    return r;
}
// Eight E2M1 values (one 32-bit word, lowest nibble first) -> four packed fp16 pairs.
__device__ __forceinline__ void cvt_e2m1x8_to_f16x2x4(uint32_t word, uint32_t (&h)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(word));
}
// Two E4M3 values (first in the low byte) -> two fp16 values.
__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint16_t two) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(two));
    return r;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// two floats -> packed bf16 (lo in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t mul_f16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// ---------------------------------------------------------------------- MMA
// All issued by one thread.  `accumulate` = 0 overwrites the accumulator, 1 adds to it.

__device__ __forceinline__ void umma_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// A from tensor memory (128 lanes x 8 columns of packed 16-bit pairs per K = 16), B from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// Block-scaled NVFP4: D (+)= (A*SFA)(B*SFB), one E4M3 scale per 16 values along K; the scale
// factors sit in tensor memory at `sfa` / `sfb`.
__device__ __forceinline__ void umma_nvf4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
// Pair (2-CTA) forms: issued by one thread of the leader CTA; the 256-row operand A and the N-wide
// operand B are taken half from each CTA's shared memory, each CTA accumulates its 128 rows.
__device__ __forceinline__ void umma_f16_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_nvf4_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}

// Shared -> tensor memory copy of one scale-factor atom: 32 rows x 128 bit, replicated into all
// four 32-lane quarters.  One thread issues it; it is ordered before later MMAs of that thread.
__device__ __forceinline__ void tc_copy_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Full cluster barrier (all threads of all CTAs of the cluster).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Barrier among `count` threads of this CTA (ids 1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

}  // namespace blz
