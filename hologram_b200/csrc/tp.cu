// Tensor-parallel all-reduce over NCCL (NVLink 5 / NVSwitch). The reference is single-device
// and has no collective; this is the sum after the row-parallel o-proj / down-proj matmuls.
// NCCL is bound at run time with dlopen so the library loads (and every single-GPU path
// runs) on a host without NCCL.
#include <dlfcn.h>
#include <string.h>

#include "common.h"

namespace {

typedef struct { char internal[128]; } NcclUniqueId;
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(void**, int, NcclUniqueId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*CommDestroyFn)(void*);
typedef const char* (*GetErrorStringFn)(int);

struct Nccl {
    void* lib = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    AllReduceFn all_reduce = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GetErrorStringFn get_error_string = nullptr;
};

Nccl* nccl() {
    static Nccl n;
    static bool tried = false;
    if (!tried) {
        tried = true;
        n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (n.lib) {
            n.get_unique_id = (GetUniqueIdFn)dlsym(n.lib, "ncclGetUniqueId");
            n.comm_init_rank = (CommInitRankFn)dlsym(n.lib, "ncclCommInitRank");
            n.all_reduce = (AllReduceFn)dlsym(n.lib, "ncclAllReduce");
            n.comm_destroy = (CommDestroyFn)dlsym(n.lib, "ncclCommDestroy");
            n.get_error_string = (GetErrorStringFn)dlsym(n.lib, "ncclGetErrorString");
        }
    }
    if (!n.lib || !n.get_unique_id || !n.comm_init_rank || !n.all_reduce || !n.comm_destroy) return nullptr;
    return &n;
}

int32_t nccl_fail(Nccl* n, int rc, const char* where) {
    return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: NCCL error %d (%s) at %s", rc,
                     n->get_error_string ? n->get_error_string(rc) : "?", where);
}

}  // namespace

extern "C" int32_t holo_b200_nccl_unique_id(uint8_t out128[128]) {
    Nccl* n = nccl();
    if (!n) return holo_fail(HOLO_ERR_INIT, "backend init failed: libnccl.so.2 could not be loaded");
    NcclUniqueId id;
    int rc = n->get_unique_id(&id);
    if (rc != 0) return nccl_fail(n, rc, "ncclGetUniqueId");
    memcpy(out128, id.internal, 128);
    return HOLO_OK;
}

extern "C" int32_t holo_b200_ctx_init_tp(holo_b200_ctx* ctx, const uint8_t id128[128], int32_t rank, int32_t world) {
    if (!ctx) return holo_fail(HOLO_ERR_INIT, "null context");
    if (world < 1 || rank < 0 || rank >= world) return holo_fail(HOLO_ERR_INIT, "backend init failed: rank %d of %d", rank, world);
    if (world == 1) {
        ctx->tp_rank = 0;
        ctx->tp_world = 1;
        return HOLO_OK;
    }
    Nccl* n = nccl();
    if (!n) return holo_fail(HOLO_ERR_INIT, "backend init failed: libnccl.so.2 could not be loaded");
    HOLO_CUDA(cudaSetDevice(ctx->device));
    NcclUniqueId id;
    memcpy(id.internal, id128, 128);
    void* comm = nullptr;
    int rc = n->comm_init_rank(&comm, world, id, rank);
    if (rc != 0) return nccl_fail(n, rc, "ncclCommInitRank");
    ctx->nccl_comm = comm;
    ctx->tp_rank = rank;
    ctx->tp_world = world;
    return HOLO_OK;
}

void holo_tp_destroy(holo_b200_ctx* ctx) {
    if (ctx->nccl_comm) {
        Nccl* n = nccl();
        if (n) n->comm_destroy(ctx->nccl_comm);
        ctx->nccl_comm = nullptr;
    }
}

int32_t holo_all_reduce(holo_b200_ctx* ctx, void* buf, uint64_t count, uint8_t dtype) {
    if (ctx->tp_world <= 1 || count == 0) return HOLO_OK;
    Nccl* n = nccl();
    if (!n || !ctx->nccl_comm) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: all_reduce without a tensor-parallel group");
    // ncclDataType_t: ncclFloat16 = 6, ncclFloat32 = 7, ncclBfloat16 = 9; ncclSum = 0
    int dt = dtype == HOLO_DTYPE_F32 ? 7 : dtype == HOLO_DTYPE_F16 ? 6 : 9;
    int rc = n->all_reduce(buf, buf, (size_t)count, dt, 0, ctx->nccl_comm, ctx->stream);
    if (rc != 0) return nccl_fail(n, rc, "ncclAllReduce");
    return HOLO_OK;
}
