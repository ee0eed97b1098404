// sharded.cu -- the column-sharded GEMM across the GPUs of one box behind the C ABI: shard arithmetic, the
// per-rank plan, and the optional exchange of the output (none / NCCL all-gather / peer stores fused into the
// GEMM epilogue).  One process per GPU; the caller moves the few bytes the ranks have to tell each other
// (a 128-byte NCCL id, 64-byte buffer handles) over whatever channel it already has.
//
// Blaze has no multi-GPU code (no NCCL, cudaSetDevice or peer copy anywhere in its tree); the entry points
// follow the create / execute / destroy triple of its plans (include/gemm/fp4_blkscaled_gemm_sm100.cuh:198-208).
// NCCL is looked up at run time (dlopen), so the library neither links nor needs it unless that exchange is asked for.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

#include "../../include/blaze_b200.h"

namespace {

// ---- the five NCCL calls this file makes, by their public C signatures
struct NcclId { char bytes[128]; };                    // ncclUniqueId
using NcclComm = void*;                                // ncclComm_t
constexpr int kNcclUint8 = 1;                          // ncclDataType_t: ncclUint8 (the gather moves bytes)
struct NcclApi {
    int (*GetUniqueId)(NcclId*);
    int (*CommInitRank)(NcclComm*, int, NcclId, int);
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t);
    int (*CommDestroy)(NcclComm);
    const char* (*GetErrorString)(int);
    bool ok = false;
    char error[200] = "";
};

NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* path = getenv("BLZ_NCCL_LIBRARY");
        void* h = dlopen((path && *path) ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) { snprintf(api.error, sizeof(api.error), "NCCL not found: %s", dlerror()); return; }
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.AllGather && api.CommDestroy;
        if (!api.ok) snprintf(api.error, sizeof(api.error), "NCCL library lacks a required symbol");
    });
    return api;
}

thread_local char g_sharded_error[256] = "";

int out_elem_bytes(int dt) { return dt == BLZ_F32 ? 4 : 2; }

}  // namespace

struct blz_sharded_plan {
    blz_sharded_desc desc;
    int64_t lo = 0, hi = 0;                 // output columns of this rank
    blz_gemm_plan* gemm = nullptr;          // (M, hi - lo, K) on this rank's weights
    NcclComm comm = nullptr;
    void* c_local = nullptr;                // NCCL exchange: this rank's [M, n_local] block (plan-owned)
    void* out_own = nullptr;                // peer stores: this rank's full-width [M, N] output (plan-owned, peer-visible)
    void* dst[8] = {};                      // peer stores: every rank's full-width output as seen from here
    bool connected = false;
    int64_t out_bytes = 0;
};

extern "C" {

const char* blz_sharded_last_error(void) { return g_sharded_error; }

blz_status blz_shard_bounds(int64_t n_total, int32_t world, int32_t rank, int32_t multiple, int64_t* lo, int64_t* hi) {
    if (!lo || !hi || n_total <= 0 || world < 1 || rank < 0 || rank >= world || multiple < 1) return BLZ_ERR_INVALID_ARGUMENT;
    // equal shards of whole tiles: every rank runs the same single-GPU kernel on full tiles
    if (n_total % world != 0 || (n_total / world) % multiple != 0) return BLZ_ERR_INVALID_ARGUMENT;
    const int64_t per = n_total / world;
    *lo = rank * per;
    *hi = (rank + 1) * per;
    return BLZ_OK;
}

blz_status blz_nccl_unique_id(uint8_t* id128) {
    if (!id128) return BLZ_ERR_INVALID_ARGUMENT;
    NcclApi& api = nccl();
    if (!api.ok) { snprintf(g_sharded_error, sizeof(g_sharded_error), "%s", api.error); return BLZ_ERR_UNSUPPORTED; }
    NcclId id;
    const int r = api.GetUniqueId(&id);
    if (r != 0) { snprintf(g_sharded_error, sizeof(g_sharded_error), "ncclGetUniqueId: %s", api.GetErrorString ? api.GetErrorString(r) : "error"); return BLZ_ERR_CUDA; }
    memcpy(id128, id.bytes, 128);
    return BLZ_OK;
}

blz_status blz_sharded_plan_create(const blz_sharded_desc* desc, blz_sharded_plan** out_plan) {
    if (!out_plan) return BLZ_ERR_INVALID_ARGUMENT;
    *out_plan = nullptr;
    if (!desc) return BLZ_ERR_INVALID_ARGUMENT;
    if (desc->world < 1 || desc->world > 8 || desc->rank < 0 || desc->rank >= desc->world) return BLZ_ERR_INVALID_ARGUMENT;
    if (desc->exchange < BLZ_EXCHANGE_NONE || desc->exchange > BLZ_EXCHANGE_PEER_STORES) return BLZ_ERR_INVALID_ARGUMENT;
    const blz_gemm_desc& g = desc->gemm;
    if (g.M <= 0 || g.N <= 0 || g.K <= 0) return BLZ_ERR_INVALID_ARGUMENT;
    if (g.b_layout != BLZ_B_KMAJOR) return BLZ_ERR_UNSUPPORTED;              // a shard is a block of rows of the K-major weights
    if (g.epilogue == BLZ_EPI_SWIGLU || g.epilogue == BLZ_EPI_RESIDUAL_ADD) return BLZ_ERR_UNSUPPORTED;
    int64_t lo = 0, hi = 0;
    blz_status s = blz_shard_bounds(g.N, desc->world, desc->rank, 128, &lo, &hi);
    if (s) return s;
    if (desc->exchange == BLZ_EXCHANGE_NCCL && desc->world > 1 && !desc->nccl_id) return BLZ_ERR_INVALID_ARGUMENT;

    blz_sharded_plan* p = new (std::nothrow) blz_sharded_plan();
    if (!p) return BLZ_ERR_OUT_OF_MEMORY;
    p->desc = *desc;
    p->lo = lo; p->hi = hi;
    auto fail = [&](blz_status st) { blz_sharded_plan_destroy(p); return st; };

    // the local problem: this rank's rows of the weights (the caller passes its shard), N = the shard's width
    blz_gemm_desc local = g;
    local.N = static_cast<int32_t>(hi - lo);
    local.ldc = 0;
    if ((s = blz_gemm_plan_create(&local, &p->gemm))) return fail(s);

    const int eb = out_elem_bytes(g.out_dtype);
    const int64_t n_local = hi - lo;
    if (desc->exchange == BLZ_EXCHANGE_NCCL && desc->world > 1) {
        NcclApi& api = nccl();
        if (!api.ok) { snprintf(g_sharded_error, sizeof(g_sharded_error), "%s", api.error); return fail(BLZ_ERR_UNSUPPORTED); }
        NcclId id;
        memcpy(id.bytes, desc->nccl_id, 128);
        const int r = api.CommInitRank(&p->comm, desc->world, id, desc->rank);
        if (r != 0) { snprintf(g_sharded_error, sizeof(g_sharded_error), "ncclCommInitRank: %s", api.GetErrorString ? api.GetErrorString(r) : "error"); p->comm = nullptr; return fail(BLZ_ERR_CUDA); }
        if (cudaMalloc(&p->c_local, static_cast<size_t>(g.M) * n_local * eb) != cudaSuccess) { (void)cudaGetLastError(); return fail(BLZ_ERR_OUT_OF_MEMORY); }
    }
    if (desc->exchange == BLZ_EXCHANGE_PEER_STORES) {
        p->out_bytes = static_cast<int64_t>(g.M) * g.N * eb;
        uint8_t handle[64];
        if ((s = blz_peer_buffer_create(p->out_bytes, &p->out_own, handle))) return fail(s);
        p->dst[desc->rank] = p->out_own;
        p->connected = desc->world == 1;
    }
    *out_plan = p;
    return BLZ_OK;
}

blz_status blz_sharded_plan_info(const blz_sharded_plan* p, blz_sharded_info* info) {
    if (!p || !info) return BLZ_ERR_INVALID_ARGUMENT;
    memset(info, 0, sizeof(*info));
    info->col_lo = p->lo; info->col_hi = p->hi;
    info->exchange = p->desc.exchange;
    info->world = p->desc.world; info->rank = p->desc.rank;
    info->own_output = p->out_own;
    return blz_gemm_plan_info(p->gemm, &info->gemm);
}

blz_status blz_sharded_plan_output_handle(blz_sharded_plan* p, uint8_t* handle64) {
    if (!p || !handle64 || !p->out_own) return BLZ_ERR_INVALID_ARGUMENT;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p->out_own) != cudaSuccess) { (void)cudaGetLastError(); return BLZ_ERR_CUDA; }
    memcpy(handle64, &h, 64);
    return BLZ_OK;
}

blz_status blz_sharded_plan_connect(blz_sharded_plan* p, const uint8_t* handles) {
    if (!p || !handles || !p->out_own) return BLZ_ERR_INVALID_ARGUMENT;
    if (p->connected) return BLZ_OK;
    for (int r = 0; r < p->desc.world; ++r) {
        if (r == p->desc.rank) continue;
        blz_status s = blz_peer_buffer_open(handles + 64 * r, &p->dst[r]);
        if (s) return s;
    }
    p->connected = true;
    return BLZ_OK;
}

blz_status blz_sharded_plan_execute(blz_sharded_plan* p, void* C, void* stream) {
    if (!p) return BLZ_ERR_INVALID_ARGUMENT;
    const blz_gemm_desc& g = p->desc.gemm;
    const int eb = out_elem_bytes(g.out_dtype);
    const int64_t n_local = p->hi - p->lo;
    switch (p->desc.exchange) {
        case BLZ_EXCHANGE_NONE:
            // C: this rank's [M, n_local] block
            if (!C) return BLZ_ERR_INVALID_ARGUMENT;
            return blz_gemm_execute(p->gemm, C, stream);
        case BLZ_EXCHANGE_NCCL: {
            // C: [world][M][n_local], rank blocks one after the other (what ncclAllGather produces)
            if (!C) return BLZ_ERR_INVALID_ARGUMENT;
            if (p->desc.world == 1) return blz_gemm_execute(p->gemm, C, stream);
            blz_status s = blz_gemm_execute(p->gemm, p->c_local, stream);
            if (s) return s;
            const int r = nccl().AllGather(p->c_local, C, static_cast<size_t>(g.M) * n_local * eb, kNcclUint8, p->comm, static_cast<cudaStream_t>(stream));
            if (r != 0) { snprintf(g_sharded_error, sizeof(g_sharded_error), "ncclAllGather: %s", nccl().GetErrorString ? nccl().GetErrorString(r) : "error"); return BLZ_ERR_CUDA; }
            return BLZ_OK;
        }
        case BLZ_EXCHANGE_PEER_STORES:
            // every rank's epilogue stores its column block into every rank's plan-owned [M, N] output; C is unused
            if (!p->connected) return BLZ_ERR_INVALID_ARGUMENT;
            return blz_gemm_execute_gather(p->gemm, p->desc.world, p->dst, g.N, p->lo, stream);
    }
    return BLZ_ERR_INVALID_ARGUMENT;
}

blz_status blz_sharded_plan_check(blz_sharded_plan* p, void* stream) {
    if (!p) return BLZ_ERR_INVALID_ARGUMENT;
    return blz_gemm_plan_check(p->gemm, stream);
}

blz_status blz_sharded_plan_destroy(blz_sharded_plan* p) {
    if (!p) return BLZ_OK;
    (void)cudaDeviceSynchronize();
    (void)cudaGetLastError();
    for (int r = 0; r < 8; ++r)
        if (p->dst[r] && p->dst[r] != p->out_own) blz_peer_buffer_close(p->dst[r]);
    if (p->out_own) blz_peer_buffer_destroy(p->out_own);
    if (p->c_local) cudaFree(p->c_local);
    if (p->comm && nccl().ok) nccl().CommDestroy(p->comm);
    blz_gemm_plan_destroy(p->gemm);
    (void)cudaGetLastError();
    delete p;
    return BLZ_OK;
}

}  // extern "C"
