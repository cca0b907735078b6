// Tensor-parallel all-reduce (NVLink 5 / NVSwitch). The reference is single-device and has no
// collective; this is the sum after the row-parallel o-proj / down-proj matmuls, optionally with
// the residual add that follows it folded in.
//
// Two transports. NCCL (bound at run time with dlopen, so the library loads and every
// single-GPU path runs on a host without it) sets up the group and carries messages over 1 MiB.
// Decode-sized messages (64 x 4096 bf16 = 512 KiB) are latency-bound, so they go through the
// library's own kernel over peer memory instead (see "peer-memory transport" below): every rank
// owns a mailbox (cudaMalloc + CUDA IPC, opened by all peers at group set-up) that its peers
// write into with plain stores over NVLink; data and ready-flag travel in the same 16-byte store.
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.h"
#include "numerics.cuh"
#include "p2p.cuh"

namespace {

typedef struct { char internal[128]; } NcclUniqueId;
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(void**, int, NcclUniqueId, int);
// ncclConfig_t as NCCL 2.17 laid it out; later versions only append fields and read `size` / `version` to know
// how much the caller filled in
struct NcclConfig {
    size_t size;
    unsigned int magic, version;
    int blocking, cga_cluster_size, min_ctas, max_ctas;
    const char* net_name;
    int split_share;
};
typedef int (*CommInitRankConfigFn)(void**, int, NcclUniqueId, int, NcclConfig*);
typedef int (*CommGetAsyncErrorFn)(void*, int*);
typedef int (*CommAbortFn)(void*);
constexpr int NCCL_IN_PROGRESS = 7;
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*CommDestroyFn)(void*);
typedef const char* (*GetErrorStringFn)(int);

struct Nccl {
    void* lib = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    AllReduceFn all_reduce = nullptr;
    AllGatherFn all_gather = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GetErrorStringFn get_error_string = nullptr;
    CommInitRankConfigFn comm_init_rank_config = nullptr;
    CommGetAsyncErrorFn comm_get_async_error = nullptr;
    CommAbortFn comm_abort = nullptr;
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
            n.all_gather = (AllGatherFn)dlsym(n.lib, "ncclAllGather");
            n.comm_destroy = (CommDestroyFn)dlsym(n.lib, "ncclCommDestroy");
            n.get_error_string = (GetErrorStringFn)dlsym(n.lib, "ncclGetErrorString");
            n.comm_init_rank_config = (CommInitRankConfigFn)dlsym(n.lib, "ncclCommInitRankConfig");
            n.comm_get_async_error = (CommGetAsyncErrorFn)dlsym(n.lib, "ncclCommGetAsyncError");
            n.comm_abort = (CommAbortFn)dlsym(n.lib, "ncclCommAbort");
        }
    }
    if (!n.lib || !n.get_unique_id || !n.comm_init_rank || !n.all_reduce || !n.comm_destroy) return nullptr;
    return &n;
}

// ---- peer-memory transport --------------------------------------------------------------------
// Message of n 16-bit elements = n/4 units of four elements; rank j owns the j-th of W equal
// slices. A unit travels as one 16-byte store {lo32, epoch, hi32, epoch}: each 8-byte half
// carries its own flag, so a reader that sees the epoch in both halves has the data, with no
// fence and no separate flag write (the data IS the signal). Three phases per thread:
//   1. scatter: push my partial of every other rank's slice into that rank's mailbox
//   2. reduce:  for my slice, poll the W-1 incoming partials, sum in rank order in f32, truncate,
//               add the residual, truncate; store locally and push the result to every peer
//   3. gather:  poll the W-1 incoming result slices and store them
// With two ranks the whole partial is pushed instead and each rank reduces the full message (one
// NVLink hop instead of two). Phase 1 never waits, phase 2 waits only for phase 1 of peers, phase 3 only for their phase 2:
// no cycle. Every poll is bounded. A mailbox region is rewritten one epoch later, which a rank
// reaches only after it has received (hence the peer has finished reading) everything of this one.
constexpr uint32_t P2P_THREADS = 256;
constexpr uint32_t P2P_MAX_CTAS = 64;

struct P2PParams {
    const uint16_t* partial;   // local, [n] 16-bit floats
    const uint16_t* residual;  // local or null
    uint16_t* out;             // local (may alias partial)
    uint8_t* mailbox[8];       // mailbox[r] = rank r's mailbox as mapped in this process
    uint32_t* state;           // local: [0] = epochs completed, [1] = CTAs finished in this launch
    uint32_t* status;
    uint32_t units_per_slice;  // n / 4 / world
    uint32_t one_shot;         // two ranks: push the whole partial, reduce everything locally (one NVLink hop instead of two)
    uint32_t wait_limit;       // polls of one unit before a thread gives up
    int rank, world, dtype;
};

// One rank's part of the all-reduce, run by `nctas` CTAs of which this is number `cta`.
__device__ __forceinline__ void all_reduce_p2p_body(const P2PParams& p, uint32_t cta, uint32_t nctas) {
    const uint32_t T = nctas * P2P_THREADS, t = cta * P2P_THREADS + threadIdx.x;
    const uint32_t U = p.units_per_slice, W = (uint32_t)p.world, me = (uint32_t)p.rank;
    const uint32_t epoch = p.state[0] + 1;
    const uint2* part2 = reinterpret_cast<const uint2*>(p.partial);
    const uint2* res2 = reinterpret_cast<const uint2*>(p.residual);
    uint2* out2 = reinterpret_cast<uint2*>(p.out);
    bool ok = true;

    if (p.one_shot) {
        // every unit is handled by the same thread in both steps, so `out` may alias `partial`
        // The buffer alternates with the epoch: a peer may still be reading my previous message when
        // I start the next one (nothing here makes me wait for its reads), but not the one before
        // that, because I cannot finish an epoch before the peer has started it.
        const uint32_t N = W * U;
        const uint64_t region = p2p_oneshot_offset(epoch);
        for (uint32_t unit = t; unit < N; unit += T) {
            const uint2 d = part2[unit];
            for (uint32_t k = 1; k < W; ++k) ll_store(p.mailbox[(me + k) % W] + region, (uint64_t)me * N + unit, d, epoch);
        }
        uint8_t* mine = p.mailbox[me] + region;
        for (uint32_t unit = t; unit < N && ok; unit += T) {
            const uint2 own = part2[unit];
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (uint32_t r = 0; r < W && ok; ++r) {
                uint2 v = own;
                if (r != me) ok = ll_load(mine, (uint64_t)r * N + unit, epoch, &v, p.wait_limit);
                acc[0] = __fadd_rn(acc[0], holo::widen16((uint16_t)(v.x & 0xffffu), p.dtype));
                acc[1] = __fadd_rn(acc[1], holo::widen16((uint16_t)(v.x >> 16), p.dtype));
                acc[2] = __fadd_rn(acc[2], holo::widen16((uint16_t)(v.y & 0xffffu), p.dtype));
                acc[3] = __fadd_rn(acc[3], holo::widen16((uint16_t)(v.y >> 16), p.dtype));
            }
            if (!ok) break;
            uint16_t h[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) h[x] = holo::narrow16(acc[x], p.dtype);
            if (res2) {
                const uint2 rv = res2[unit];
                const uint16_t rr[4] = {(uint16_t)(rv.x & 0xffffu), (uint16_t)(rv.x >> 16), (uint16_t)(rv.y & 0xffffu), (uint16_t)(rv.y >> 16)};
#pragma unroll
                for (int x = 0; x < 4; ++x) h[x] = holo::narrow16(__fadd_rn(holo::widen16(h[x], p.dtype), holo::widen16(rr[x], p.dtype)), p.dtype);
            }
            out2[unit] = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
        }
    } else {
    // my slice's partials first: phase 2 may write `out` over them when out aliases partial only
    // at the same unit, which is read before it is written
    // 1. scatter
    for (uint32_t idx = t; idx < (W - 1) * U; idx += T) {
        const uint32_t j = (me + 1 + idx / U) % W, u = idx % U;
        ll_store(p.mailbox[j], (uint64_t)me * U + u, part2[(uint64_t)j * U + u], epoch);
    }
    // 2. reduce my slice
    uint8_t* box = p.mailbox[me];
    for (uint32_t u = t; u < U && ok; u += T) {
        const uint2 own = part2[(uint64_t)me * U + u];
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t r = 0; r < W && ok; ++r) {
            uint2 v = own;
            if (r != me) ok = ll_load(box, (uint64_t)r * U + u, epoch, &v, p.wait_limit);
            acc[0] = __fadd_rn(acc[0], holo::widen16((uint16_t)(v.x & 0xffffu), p.dtype));
            acc[1] = __fadd_rn(acc[1], holo::widen16((uint16_t)(v.x >> 16), p.dtype));
            acc[2] = __fadd_rn(acc[2], holo::widen16((uint16_t)(v.y & 0xffffu), p.dtype));
            acc[3] = __fadd_rn(acc[3], holo::widen16((uint16_t)(v.y >> 16), p.dtype));
        }
        if (!ok) break;
        uint16_t h[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) h[x] = holo::narrow16(acc[x], p.dtype);
        if (res2) {
            const uint2 rv = res2[(uint64_t)me * U + u];
            const uint16_t rr[4] = {(uint16_t)(rv.x & 0xffffu), (uint16_t)(rv.x >> 16), (uint16_t)(rv.y & 0xffffu), (uint16_t)(rv.y >> 16)};
#pragma unroll
            for (int x = 0; x < 4; ++x) h[x] = holo::narrow16(__fadd_rn(holo::widen16(h[x], p.dtype), holo::widen16(rr[x], p.dtype)), p.dtype);
        }
        const uint2 res = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
        out2[(uint64_t)me * U + u] = res;
        for (uint32_t k = 1; k < W; ++k) ll_store(p.mailbox[(me + k) % W] + P2P_REGION_BYTES, (uint64_t)me * U + u, res, epoch);
    }
    // 3. gather the other slices' results
    for (uint32_t idx = t; idx < (W - 1) * U && ok; idx += T) {
        const uint32_t r = (me + 1 + idx / U) % W, u = idx % U;
        uint2 v;
        ok = ll_load(box + P2P_REGION_BYTES, (uint64_t)r * U + u, epoch, &v, p.wait_limit);
        if (ok) out2[(uint64_t)r * U + u] = v;
    }
    }
    if (!ok) atomicOr(p.status, 8u);
    // the launch's last CTA advances the epoch (every CTA has read it by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t done = atomicAdd(p.state + 1, 1u);
        if (done == nctas - 1) {
            p.state[1] = 0;
            p.state[0] = epoch;
        }
    }
}

__global__ void __launch_bounds__(P2P_THREADS) all_reduce_p2p_kernel(const P2PParams p) {
    holo_pdl_trigger();
    holo_pdl_wait();
    all_reduce_p2p_body(p, blockIdx.x, gridDim.x);
}

// All ranks of a group as one cooperative launch on one GPU (grid.y = rank): the same device code
// with every mailbox in local memory. Lets the protocol be run for any world size on a single GPU;
// the ranks' CTAs wait on one another, hence the cooperative launch (all CTAs co-resident).
struct P2PEmulation {
    P2PParams rank[8];
    int withheld;   // this emulated rank never sends (its CTAs return at once): what a dead peer looks like to the others
};
__global__ void __launch_bounds__(P2P_THREADS) all_reduce_p2p_emulation_kernel(const P2PEmulation e) {
    if ((int)blockIdx.y == e.withheld) return;
    all_reduce_p2p_body(e.rank[blockIdx.y], blockIdx.x, gridDim.x);
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

namespace {
// Wait until a non-blocking communicator has finished what it was asked to do. Returns the NCCL result
// (0 = done), or -1 when `timeout_ms` ran out first (the caller aborts the communicator).
int nccl_wait(Nccl* n, void* comm, uint32_t timeout_ms) {
    if (!n->comm_get_async_error) return 0;
    struct timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        int state = 0;
        const int rc = n->comm_get_async_error(comm, &state);
        if (rc != 0) return rc;
        if (state != NCCL_IN_PROGRESS) return state;
        struct timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        const uint64_t ms = (uint64_t)(t1.tv_sec - t0.tv_sec) * 1000u + (uint64_t)((t1.tv_nsec - t0.tv_nsec) / 1000000);
        if (timeout_ms && ms >= timeout_ms) return -1;
        struct timespec nap = {0, 2 * 1000 * 1000};
        nanosleep(&nap, nullptr);
    }
}
}  // namespace

extern "C" int32_t holo_b200_ctx_init_tp(holo_b200_ctx* ctx, const uint8_t id128[128], int32_t rank, int32_t world) {
    uint32_t timeout_ms = 120000;
    if (const char* e = getenv("HOLO_TP_INIT_TIMEOUT_MS")) timeout_ms = (uint32_t)atoll(e);
    return holo_b200_ctx_init_tp_timeout(ctx, id128, rank, world, timeout_ms);
}

extern "C" int32_t holo_b200_ctx_init_tp_timeout(holo_b200_ctx* ctx, const uint8_t id128[128], int32_t rank, int32_t world, uint32_t timeout_ms) {
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
    int rc;
    const bool nonblocking = n->comm_init_rank_config && n->comm_get_async_error && n->comm_abort && !getenv("HOLO_TP_BLOCKING_INIT");
    if (nonblocking) {
        // Non-blocking set-up with a host-side time limit: the group forms over the bootstrap network before
        // anything is enqueued on a GPU, so a rank that never joins (or joins with another world size) is a
        // host timeout here, followed by an abort of the half-made communicator, never a hung collective.
        NcclConfig cfg;
        memset(&cfg, 0, sizeof cfg);
        cfg.size = sizeof cfg;
        cfg.magic = 0xcafebeef;
        cfg.version = 2 * 10000 + 17 * 100;   // NCCL_VERSION(2, 17, 0): the layout filled in here
        cfg.blocking = 0;
        cfg.cga_cluster_size = cfg.min_ctas = cfg.max_ctas = cfg.split_share = (int)0x80000000;   // NCCL_CONFIG_UNDEF_INT
        cfg.net_name = nullptr;
        rc = n->comm_init_rank_config(&comm, world, id, rank, &cfg);
        if (rc != 0 && rc != NCCL_IN_PROGRESS) return nccl_fail(n, rc, "ncclCommInitRankConfig");
        rc = nccl_wait(n, comm, timeout_ms);
        if (rc != 0) {
            if (comm) n->comm_abort(comm);
            if (rc == -1)
                return holo_fail(HOLO_ERR_INIT, "backend init failed: the tensor-parallel group of %d ranks did not form within %u ms (rank %d waited; "
                                 "a rank is missing or was given another world size)", world, timeout_ms, rank);
            return nccl_fail(n, rc, "ncclCommInitRankConfig (asynchronous)");
        }
        ctx->nccl_nonblocking = true;
    } else {
        rc = n->comm_init_rank(&comm, world, id, rank);
        if (rc != 0) return nccl_fail(n, rc, "ncclCommInitRank");
    }
    ctx->nccl_comm = comm;
    ctx->tp_rank = rank;
    ctx->tp_world = world;
    // Peer-memory mailboxes. Every rank of the group takes part in the two collectives below whatever its own
    // outcome was (transport switched off by HOLO_TP_P2P=0, IPC not permitted, an allocation that failed): a rank
    // that skipped one would leave its peers waiting inside it. The ranks agree on the transport through a
    // min-reduce of "my set-up worked", so one rank's "no" switches all of them to NCCL.
    const char* env = getenv("HOLO_TP_P2P");
    const bool want = world <= 8 && n->all_gather && !(env && atoi(env) == 0);
    uint8_t* mine = nullptr;
    uint8_t* dev_handles = nullptr;
    cudaIpcMemHandle_t handles[8];
    cudaIpcMemHandle_t h;
    memset(&h, 0, sizeof h);
    // the exchange buffer is needed by every rank: without it this rank cannot take part, and init fails here,
    // before any collective (the peers' set-up then runs into its own time limit instead of a hung kernel)
    if (cudaMalloc(&dev_handles, 8 * sizeof(cudaIpcMemHandle_t)) != cudaSuccess) {
        cudaGetLastError();
        return holo_fail(HOLO_ERR_INIT, "backend init failed: tensor-parallel set-up could not allocate device memory");
    }
    bool ok = want;
    // cleared on the context's stream and waited for before any peer can learn the address
    if (ok) ok = cudaMalloc(&mine, P2P_MAILBOX_BYTES) == cudaSuccess && cudaMemsetAsync(mine, 0, P2P_MAILBOX_BYTES, ctx->stream) == cudaSuccess &&
                 cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    if (ok) ok = cudaIpcGetMemHandle(&h, mine) == cudaSuccess;
    bool collectives_ok = true;
    if (n->all_gather) {
        cudaMemcpy(dev_handles + (size_t)rank * sizeof h, &h, sizeof h, cudaMemcpyHostToDevice);
        rc = n->all_gather(dev_handles + (size_t)rank * sizeof h, dev_handles, sizeof h, /*ncclInt8*/ 0, comm, ctx->stream);
        if (ctx->nccl_nonblocking && (rc == 0 || rc == NCCL_IN_PROGRESS)) rc = nccl_wait(n, comm, timeout_ms);
        if (rc != 0 || cudaStreamSynchronize(ctx->stream) != cudaSuccess) collectives_ok = false;
        if (cudaMemcpy(handles, dev_handles, world * sizeof h, cudaMemcpyDeviceToHost) != cudaSuccess) ok = false;
    } else {
        ok = false;
    }
    if (!collectives_ok) {
        cudaFree(dev_handles);
        if (mine) cudaFree(mine);
        cudaGetLastError();
        return holo_fail(HOLO_ERR_INIT, "backend init failed: the handle exchange of the tensor-parallel group did not complete (NCCL result %d)", rc);
    }
    if (ok) {
        for (int r = 0; r < world && ok; ++r) {
            if (r == rank) {
                ctx->tp_mailbox[r] = mine;
            } else {
                void* q = nullptr;
                ok = cudaIpcOpenMemHandle(&q, handles[r], cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
                ctx->tp_mailbox[r] = (uint8_t*)q;
            }
        }
    }
    if (ok) ok = cudaMalloc(&ctx->tp_epochs, 256) == cudaSuccess && cudaMemsetAsync(ctx->tp_epochs, 0, 256, ctx->stream) == cudaSuccess &&
                 cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    cudaGetLastError();  // a failed attempt above must not poison later launches
    {
        float flag = ok ? 1.0f : 0.0f;
        cudaMemcpy(dev_handles, &flag, 4, cudaMemcpyHostToDevice);
        rc = n->all_reduce(dev_handles, dev_handles, 1, /*ncclFloat32*/ 7, /*ncclMin*/ 3, comm, ctx->stream);
        if (ctx->nccl_nonblocking && (rc == 0 || rc == NCCL_IN_PROGRESS)) rc = nccl_wait(n, comm, timeout_ms);
        if (rc != 0 || cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
            cudaFree(dev_handles);
            return nccl_fail(n, rc, "ncclAllReduce (transport agreement)");
        }
        cudaMemcpy(&flag, dev_handles, 4, cudaMemcpyDeviceToHost);
        ok = flag > 0.5f;
        cudaFree(dev_handles);
    }
    ctx->tp_p2p = ok;
    if (!ok) {
        for (int r = 0; r < world; ++r)
            if (r != rank && ctx->tp_mailbox[r]) cudaIpcCloseMemHandle(ctx->tp_mailbox[r]);
        memset(ctx->tp_mailbox, 0, sizeof ctx->tp_mailbox);
        if (mine) cudaFree(mine);
        if (ctx->tp_epochs) cudaFree(ctx->tp_epochs);
        ctx->tp_epochs = nullptr;
        cudaGetLastError();
    }
    return HOLO_OK;
}

extern "C" int32_t holo_b200_ctx_tp_transport(holo_b200_ctx* ctx) {
    if (!ctx || ctx->tp_world <= 1) return 0;
    return ctx->tp_p2p ? 2 : 1;
}

void holo_tp_destroy(holo_b200_ctx* ctx) {
    if (ctx->tp_p2p) {
        for (int r = 0; r < ctx->tp_world; ++r) {
            if (!ctx->tp_mailbox[r]) continue;
            if (r == ctx->tp_rank) cudaFree(ctx->tp_mailbox[r]);
            else cudaIpcCloseMemHandle(ctx->tp_mailbox[r]);
            ctx->tp_mailbox[r] = nullptr;
        }
        if (ctx->tp_epochs) cudaFree(ctx->tp_epochs);
        ctx->tp_epochs = nullptr;
        ctx->tp_p2p = false;
    }
    if (ctx->nccl_comm) {
        Nccl* n = nccl();
        if (n) n->comm_destroy(ctx->nccl_comm);
        ctx->nccl_comm = nullptr;
    }
}

// out = all_reduce(partial) (+ residual). `out` may alias `partial`; `residual` may be null.
int32_t holo_all_reduce_add(holo_b200_ctx* ctx, const void* partial, const void* residual, void* out, uint64_t count, uint8_t dtype) {
    if (count == 0) return HOLO_OK;
    const bool sixteen = dtype == HOLO_DTYPE_BF16 || dtype == HOLO_DTYPE_F16;
    // Which transport carries a message is decided by values every rank shares (dtype, count), never by a
    // local pointer: two ranks taking different routes would wait for each other for ever. A buffer that the
    // peer-memory kernel cannot take (not 8-byte aligned) is therefore refused, loudly, instead of rerouted.
    if (ctx->tp_world > 1 && ctx->tp_p2p && sixteen && count <= P2P_MAX_ELEMS && (count % (4ull * ctx->tp_world)) == 0) {
        if ((((uintptr_t)partial | (uintptr_t)residual | (uintptr_t)out) & 7u) != 0)
            return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: all_reduce operands must be 8-byte aligned on the peer-memory transport");
        P2PParams p;
        p.partial = (const uint16_t*)partial;
        p.residual = (const uint16_t*)residual;
        p.out = (uint16_t*)out;
        for (int r = 0; r < 8; ++r) p.mailbox[r] = ctx->tp_mailbox[r];
        p.state = ctx->tp_epochs;
        p.status = ctx->dev_status;
        p.units_per_slice = (uint32_t)(count / 4 / ctx->tp_world);
        p.one_shot = (ctx->tp_world == 2 && 4ull * ctx->tp_world * count <= P2P_ONESHOT_BYTES && !getenv("HOLO_TP_TWO_SHOT")) ? 1u : 0u;
        p.wait_limit = P2P_WAIT_LIMIT;
        p.rank = ctx->tp_rank;
        p.world = ctx->tp_world;
        p.dtype = dtype;
        // enough threads for one unit of the widest phase each, at most P2P_MAX_CTAS CTAs (all co-resident)
        const uint64_t widest = p.one_shot ? (uint64_t)p.units_per_slice * ctx->tp_world : (uint64_t)p.units_per_slice * (ctx->tp_world - 1);
        uint32_t ctas = (uint32_t)((widest + P2P_THREADS - 1) / P2P_THREADS);
        if (ctas > P2P_MAX_CTAS) ctas = P2P_MAX_CTAS;
        if (ctas < 1) ctas = 1;
        HOLO_CUDA(holo_launch_kernel(ctx, all_reduce_p2p_kernel, dim3(ctas), dim3(P2P_THREADS), 0, 1, p));
        ctx->launches++;
        return HOLO_OK;
    }
    if (out != partial)
        HOLO_CUDA(cudaMemcpyAsync(out, partial, count * holo_dtype_size(dtype), cudaMemcpyDeviceToDevice, ctx->stream));
    if (ctx->tp_world > 1) {
        Nccl* n = nccl();
        if (!n || !ctx->nccl_comm) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: all_reduce without a tensor-parallel group");
        // ncclDataType_t: ncclFloat16 = 6, ncclFloat32 = 7, ncclBfloat16 = 9; ncclSum = 0
        int dt = dtype == HOLO_DTYPE_F32 ? 7 : dtype == HOLO_DTYPE_F16 ? 6 : 9;
        int rc = n->all_reduce(out, out, (size_t)count, dt, 0, ctx->nccl_comm, ctx->stream);
        if (ctx->nccl_nonblocking && (rc == 0 || rc == NCCL_IN_PROGRESS)) rc = nccl_wait(n, ctx->nccl_comm, 60000);   // enqueue only; the kernel runs on the stream
        if (rc != 0) return nccl_fail(n, rc, "ncclAllReduce");
    }
    if (residual) return holo_launch_binary(ctx, 0, out, residual, out, count, dtype);
    return HOLO_OK;
}

int32_t holo_all_reduce(holo_b200_ctx* ctx, void* buf, uint64_t count, uint8_t dtype) {
    if (ctx->tp_world <= 1 || count == 0) return HOLO_OK;
    return holo_all_reduce_add(ctx, buf, nullptr, buf, count, dtype);
}

// Runs the peer-memory all-reduce for `world` emulated ranks on this context's GPU: partials[r] and
// outs[r] are device pointers to rank r's `count` 16-bit elements (residuals[r] may be null, outs
// may alias partials). Mailboxes are allocated for the call and freed again. For tests.
extern "C" int32_t holo_b200_tp_emulate_all_reduce(holo_b200_ctx* ctx, int32_t world, const void* const* partials, const void* const* residuals,
                                                   void* const* outs, uint64_t count, uint8_t dtype, int32_t repeats) {
    return holo_b200_tp_emulate_all_reduce_ex(ctx, world, partials, residuals, outs, count, dtype, repeats, -1, 0);
}

extern "C" int32_t holo_b200_tp_emulate_all_reduce_ex(holo_b200_ctx* ctx, int32_t world, const void* const* partials, const void* const* residuals,
                                                      void* const* outs, uint64_t count, uint8_t dtype, int32_t repeats, int32_t withheld_rank,
                                                      uint32_t poll_limit) {
    if (!ctx || world < 2 || world > 8 || !partials || !outs || withheld_rank >= world) return holo_fail(HOLO_ERR_INIT, "backend init failed: bad argument");
    if ((dtype != HOLO_DTYPE_BF16 && dtype != HOLO_DTYPE_F16) || count == 0 || count > P2P_MAX_ELEMS || (count % (4ull * world)) != 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: the peer-memory all-reduce takes 16-bit messages of at most %u elements, a multiple of 4 x world",
                         P2P_MAX_ELEMS);
    HOLO_CUDA(cudaSetDevice(ctx->device));
    uint8_t* boxes = nullptr;
    uint32_t* states = nullptr;
    // cleared on the launch stream: a memset on the default stream is not ordered with it
    HOLO_CUDA(cudaMalloc(&boxes, (size_t)world * P2P_MAILBOX_BYTES));
    HOLO_CUDA(cudaMemsetAsync(boxes, 0, (size_t)world * P2P_MAILBOX_BYTES, ctx->stream));
    HOLO_CUDA(cudaMalloc(&states, (size_t)world * 256));
    HOLO_CUDA(cudaMemsetAsync(states, 0, (size_t)world * 256, ctx->stream));
    P2PEmulation e;
    for (int r = 0; r < world; ++r) {
        P2PParams& p = e.rank[r];
        p.partial = (const uint16_t*)partials[r];
        p.residual = residuals ? (const uint16_t*)residuals[r] : nullptr;
        p.out = (uint16_t*)outs[r];
        for (int q = 0; q < 8; ++q) p.mailbox[q] = q < world ? boxes + (size_t)q * P2P_MAILBOX_BYTES : nullptr;
        p.state = states + r * 64;
        p.status = ctx->dev_status;
        p.units_per_slice = (uint32_t)(count / 4 / world);
        p.one_shot = (world == 2 && 4ull * world * count <= P2P_ONESHOT_BYTES && !getenv("HOLO_TP_TWO_SHOT")) ? 1u : 0u;
        p.wait_limit = poll_limit ? poll_limit : P2P_WAIT_LIMIT;
        p.rank = r;
        p.world = world;
        p.dtype = dtype;
    }
    const uint64_t widest = e.rank[0].one_shot ? (uint64_t)e.rank[0].units_per_slice * world : (uint64_t)e.rank[0].units_per_slice * (world - 1);
    uint32_t ctas = (uint32_t)((widest + P2P_THREADS - 1) / P2P_THREADS);
    if (ctas > P2P_MAX_CTAS) ctas = P2P_MAX_CTAS;
    if (ctas < 1) ctas = 1;
    e.withheld = withheld_rank;
    void* args[] = {&e};
    cudaError_t err = cudaSuccess;
    for (int i = 0; i < repeats && err == cudaSuccess; ++i) {
        err = cudaLaunchCooperativeKernel((const void*)all_reduce_p2p_emulation_kernel, dim3(ctas, world), dim3(P2P_THREADS), args, 0, ctx->stream);
        ctx->launches++;
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(ctx->stream);
    cudaFree(boxes);
    cudaFree(states);
    if (err != cudaSuccess) return holo_cuda_fail(err, "all_reduce_p2p_emulation_kernel");
    // a poll that ran out left its mark in the status word: report it here, as every synchronising call does
    return holo_b200_ctx_synchronize(ctx);
}
