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
                if (r != me) ok = ll_load(mine, (uint64_t)r * N + unit, epoch, &v);
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
            if (r != me) ok = ll_load(box, (uint64_t)r * U + u, epoch, &v);
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
        ok = ll_load(box + P2P_REGION_BYTES, (uint64_t)r * U + u, epoch, &v);
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
};
__global__ void __launch_bounds__(P2P_THREADS) all_reduce_p2p_emulation_kernel(const P2PEmulation e) {
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
    // Peer-memory mailboxes. Any failure here (IPC not permitted, no peer access, more than 8
    // ranks) leaves the group on NCCL alone; the ranks agree on the outcome through a min-reduce.
    const char* env = getenv("HOLO_TP_P2P");
    bool want = world <= 8 && n->all_gather && !(env && atoi(env) == 0);
    uint8_t* mine = nullptr;
    uint8_t* dev_handles = nullptr;
    cudaIpcMemHandle_t handles[8];
    bool ok = want;
    // cleared on the context's stream and waited for before any peer can learn the address
    if (ok) ok = cudaMalloc(&mine, P2P_MAILBOX_BYTES) == cudaSuccess && cudaMemsetAsync(mine, 0, P2P_MAILBOX_BYTES, ctx->stream) == cudaSuccess &&
                 cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    if (ok) ok = cudaMalloc(&dev_handles, 8 * sizeof(cudaIpcMemHandle_t)) == cudaSuccess;
    cudaIpcMemHandle_t h;
    memset(&h, 0, sizeof h);
    if (ok) ok = cudaIpcGetMemHandle(&h, mine) == cudaSuccess;
    if (dev_handles) {
        // every rank takes part in the gather, whether or not its own set-up worked
        cudaMemcpy(dev_handles + (size_t)rank * sizeof h, &h, sizeof h, cudaMemcpyHostToDevice);
        rc = n->all_gather(dev_handles + (size_t)rank * sizeof h, dev_handles, sizeof h, /*ncclInt8*/ 0, comm, ctx->stream);
        if (rc != 0 || cudaStreamSynchronize(ctx->stream) != cudaSuccess) ok = false;
        if (cudaMemcpy(handles, dev_handles, world * sizeof h, cudaMemcpyDeviceToHost) != cudaSuccess) ok = false;
    } else {
        ok = false;
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
    // agreement: min over ranks of "my set-up worked" (want == false on one rank switches all off;
    // a rank without a gather buffer cannot take part in a collective, so it has to fail init)
    if (!dev_handles && want) return holo_fail(HOLO_ERR_INIT, "backend init failed: tensor-parallel set-up could not allocate device memory");
    if (dev_handles) {
        float flag = ok ? 1.0f : 0.0f;
        cudaMemcpy(dev_handles, &flag, 4, cudaMemcpyHostToDevice);
        rc = n->all_reduce(dev_handles, dev_handles, 1, /*ncclFloat32*/ 7, /*ncclMin*/ 3, comm, ctx->stream);
        if (rc != 0 || cudaStreamSynchronize(ctx->stream) != cudaSuccess) return nccl_fail(n, rc, "ncclAllReduce (transport agreement)");
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
    const bool aligned = (((uintptr_t)partial | (uintptr_t)residual | (uintptr_t)out) & 7u) == 0;
    if (ctx->tp_world > 1 && ctx->tp_p2p && sixteen && aligned && count <= P2P_MAX_ELEMS && (count % (4ull * ctx->tp_world)) == 0) {
        P2PParams p;
        p.partial = (const uint16_t*)partial;
        p.residual = (const uint16_t*)residual;
        p.out = (uint16_t*)out;
        for (int r = 0; r < 8; ++r) p.mailbox[r] = ctx->tp_mailbox[r];
        p.state = ctx->tp_epochs;
        p.status = ctx->dev_status;
        p.units_per_slice = (uint32_t)(count / 4 / ctx->tp_world);
        p.one_shot = (ctx->tp_world == 2 && 4ull * ctx->tp_world * count <= P2P_ONESHOT_BYTES && !getenv("HOLO_TP_TWO_SHOT")) ? 1u : 0u;
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
    if (!ctx || world < 2 || world > 8 || !partials || !outs) return holo_fail(HOLO_ERR_INIT, "backend init failed: bad argument");
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
        p.rank = r;
        p.world = world;
        p.dtype = dtype;
    }
    const uint64_t widest = e.rank[0].one_shot ? (uint64_t)e.rank[0].units_per_slice * world : (uint64_t)e.rank[0].units_per_slice * (world - 1);
    uint32_t ctas = (uint32_t)((widest + P2P_THREADS - 1) / P2P_THREADS);
    if (ctas > P2P_MAX_CTAS) ctas = P2P_MAX_CTAS;
    if (ctas < 1) ctas = 1;
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
    return HOLO_OK;
}
