// A one-tile E4M3 GEMM written only with the low-level helper names of gemm/tma_utils.cuh and
// gemm/tmem_utils.cuh (the names Blaze's bring-up code uses): TMA loads of a 128x128-byte A and B
// tile, four tcgen05.mma of K = 32, accumulator back through tmem_store_to_smem_warp.
// With every byte 0x38 (E4M3 1.0) each of the 128x128 outputs must be exactly K = 128 -- the known
// answer of Blaze's own primitive test (64 for its K = 64 tile).  A second launch uses a
// position-dependent A to catch a transposed or mis-swizzled tile.
// Prints "PASS" / "FAIL ..." and returns 0 / 1.  Every wait in it is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "gemm/tma_utils.cuh"
#include "gemm/tmem_utils.cuh"

using namespace blaze;

constexpr int TM = 128, TN = 128, TK = 128;

struct __align__(1024) Smem {
    uint8_t a[TM * TK];
    uint8_t b[TN * TK];
    float c[TM * (TN + SMEM_C_PAD)];
    alignas(8) uint64_t bar_load;
    alignas(8) uint64_t bar_mma;
    uint32_t tmem_base;
};

__global__ void __launch_bounds__(128) one_tile_kernel(const __grid_constant__ TmaDescriptor da, const __grid_constant__ TmaDescriptor db, float* out) {
    extern __shared__ uint8_t raw[];
    Smem* s = reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbarrier_init(&s->bar_load, 1);
        mbarrier_init(&s->bar_mma, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&s->tmem_base, TN);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const tmem_addr_t acc = s->tmem_base;

    if (warp == 0 && elect_one_sync()) {
        mbarrier_expect_tx(&s->bar_load, tma_tile_bytes(TM, TK, 1) + tma_tile_bytes(TN, TK, 1));
        tma_load_2d(s->a, &da, 0, 0, &s->bar_load);
        tma_load_2d(s->b, &db, 0, 0, &s->bar_load);
    }
    mbarrier_wait(&s->bar_load, 0);
    if (warp == 0) {
        if (elect_one_sync()) {
            const uint32_t idesc = make_idesc_f8f6f4(0, 0, TM, TN);
            const uint32_t sa = static_cast<uint32_t>(__cvta_generic_to_shared(s->a)), sb = static_cast<uint32_t>(__cvta_generic_to_shared(s->b));
            for (int k = 0; k < TK / 32; ++k) {
                // 128-byte swizzle: eight rows per 1024-byte group, 32 bytes of K further per instruction
                const uint64_t desc_a = make_smem_desc(sa + 32 * k, 1024, 2), desc_b = make_smem_desc(sb + 32 * k, 1024, 2);
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                             ::"r"(acc), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(k) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&s->bar_mma))) : "memory");
        }
        __syncwarp();
    }
    mbarrier_wait(&s->bar_mma, 0);
    tmem_store_to_smem_warp(s->c, acc, TN, TN + SMEM_C_PAD, warp);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    for (int i = threadIdx.x; i < TM * TN; i += blockDim.x) out[i] = s->c[(i / TN) * (TN + SMEM_C_PAD) + i % TN];
    __syncthreads();
    if (warp == 0) tmem_dealloc(acc, TN);
}

static float e4m3_value(uint8_t v) {                       // positive normal codes only (what this test uses)
    const int e = (v >> 3) & 15, m = v & 7;
    float f = 1.0f + m / 8.0f;
    for (int i = 7; i < e; ++i) f *= 2.0f;
    for (int i = e; i < 7; ++i) f *= 0.5f;
    return f;
}

int main() {
    std::vector<uint8_t> ha(TM * TK, 0x38), hb(TN * TK, 0x38);
    uint8_t *da_mem = nullptr, *db_mem = nullptr;
    float* dout = nullptr;
    if (cudaMalloc(&da_mem, ha.size()) || cudaMalloc(&db_mem, hb.size()) || cudaMalloc(&dout, TM * TN * sizeof(float))) { std::printf("FAIL cudaMalloc\n"); return 1; }
    const size_t smem = sizeof(Smem) + 1024;
    cudaFuncSetAttribute(one_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    std::vector<float> hout(TM * TN);
    for (int pass = 0; pass < 2; ++pass) {
        if (pass == 1) {
            // A[m][k] = 1.0 only at k = (5 m + 3) % K, else 2^-6; B[n][k] takes four different values by (n + k) % 4
            for (int m = 0; m < TM; ++m) for (int k = 0; k < TK; ++k) ha[m * TK + k] = (k == (5 * m + 3) % TK) ? 0x38 : 0x08;
            for (int n = 0; n < TN; ++n) for (int k = 0; k < TK; ++k) hb[n * TK + k] = static_cast<uint8_t>(0x30 + 8 * ((n + k) % 4));
        }
        cudaMemcpy(da_mem, ha.data(), ha.size(), cudaMemcpyHostToDevice);
        cudaMemcpy(db_mem, hb.data(), hb.size(), cudaMemcpyHostToDevice);
        cudaMemset(dout, 0xFF, TM * TN * sizeof(float));
        TmaDescriptor ta, tb;
        create_tma_desc_2d(&ta, da_mem, CU_TENSOR_MAP_DATA_TYPE_UINT8, TM, TK, TM, TK, TmaSwizzle::B128);
        create_tma_desc_2d(&tb, db_mem, CU_TENSOR_MAP_DATA_TYPE_UINT8, TN, TK, TN, TK, TmaSwizzle::B128);
        one_tile_kernel<<<1, 128, smem>>>(ta, tb, dout);
        const cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { std::printf("FAIL %s\n", cudaGetErrorString(e)); return 1; }
        cudaMemcpy(hout.data(), dout, hout.size() * sizeof(float), cudaMemcpyDeviceToHost);
        int bad = 0;
        for (int m = 0; m < TM && bad < 5; ++m)
            for (int n = 0; n < TN && bad < 5; ++n) {
                float want = 0.0f;
                for (int k = 0; k < TK; ++k) want += e4m3_value(ha[m * TK + k]) * e4m3_value(hb[n * TK + k]);
                if (hout[m * TN + n] != want) { std::printf("FAIL pass %d C[%d][%d] = %g, expected %g\n", pass, m, n, hout[m * TN + n], want); ++bad; }
            }
        if (bad) return 1;
    }
    std::printf("PASS\n");
    return 0;
}
