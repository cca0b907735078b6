// Archive session: load a `.holo`, fuse, place every slot on the device, walk the call list.
// The device-side restatement of InferenceSession::load / execute for the served variants
// (crates/hologram-exec/src/session.rs:428-792 load, :846-932 execute, :1052-1289 walk):
//   * calls are ordered by the ExecPlan levels (one level in call order when absent, :473);
//   * load-time fusion: MatMul -> activation becomes MatMulActivation, MatMul -> Add(residual)
//     becomes MatMulAdd (fuse_matmul_epilogue, session.rs:2150-2377); the backend therefore
//     executes the fused calls, exactly as the CPU backend does;
//   * every slot is sized from the largest BufferRef / port / constant that touches it, floor
//     64 B, rounded to 64 (session.rs:544-629) and lives in HBM for the session's lifetime;
//     constants are uploaded once (pool.pin_bytes, :686);
//   * a KvCacheWrite from an input-port cache to an output port is realised as the in-place
//     move (kv_move_in_place, session.rs:1313-1370): both slots share one device buffer and
//     only the new rows are written;
//   * the walk can be captured once into a CUDA graph and replayed per step.
#include <string.h>

#include <algorithm>
#include <set>

#include "archive.h"
#include "common.h"

struct holo_b200_session {
    holo_b200_ctx* ctx = nullptr;
    holo_b200_workspace* ws = nullptr;
    HoloArchive ar;
    std::vector<HoloKernelCall> calls;  // execution order, after fusion
    uint32_t fused = 0, moved_in_place = 0;
    uint64_t device_bytes = 0;
    cudaGraphExec_t graph = nullptr;
};

namespace {

bool same_range(const HoloBufferRef& a, const HoloBufferRef& b) { return a.slot == b.slot && a.offset == b.offset; }

uint8_t fused_act_of(uint16_t kind) {  // KernelCall::fused_activation, kernel_call.rs:1283-1297 (table-backed ones)
    switch (kind) {
        case HOLO_K_GELU: return HOLO_FUSED_GELU;
        case HOLO_K_SILU: return HOLO_FUSED_SILU;
        case HOLO_K_SIGMOID: return HOLO_FUSED_SIGMOID;
        case HOLO_K_TANH: return HOLO_FUSED_TANH;
        case HOLO_K_EXP: return HOLO_FUSED_EXP;
        default: return 0;
    }
}

// fuse_matmul_epilogue: a bf16 MatMul whose output is read by exactly one later call, which is
// a table-backed activation over the whole product or an Add with the product as one operand,
// and is not itself a graph output, is folded into that consumer's position.
uint32_t fuse_matmul_epilogue(std::vector<HoloKernelCall>& calls, const std::set<uint32_t>& output_slots) {
    uint32_t fused = 0;
    std::vector<bool> dead(calls.size(), false);
    for (size_t i = 0; i < calls.size(); ++i) {
        if (dead[i] || calls[i].kind != HOLO_K_MATMUL) continue;
        const HoloMatMulCall mm = calls[i].u.matmul;
        if (mm.dtype != HOLO_DTYPE_BF16 && mm.dtype != HOLO_DTYPE_F16 && mm.dtype != HOLO_DTYPE_F32) continue;
        if (output_slots.count(mm.output.slot)) continue;
        int consumer = -1, readers = 0;
        bool clobbered = false;
        for (size_t j = i + 1; j < calls.size(); ++j) {
            if (dead[j]) continue;
            HoloKernelCall tmp = calls[j];
            HoloRefList refs;
            if (!holo_collect_refs(&tmp, &refs)) continue;
            for (int r = 0; r < refs.n; ++r) {
                if (refs.refs[r]->slot != mm.output.slot) continue;
                if (refs.written[r]) clobbered = true;
                else {
                    ++readers;
                    consumer = (int)j;
                }
            }
        }
        if (readers != 1 || clobbered || consumer < 0) continue;
        HoloKernelCall& c = calls[consumer];
        const uint64_t count = (uint64_t)mm.m * mm.n;
        const uint8_t act = fused_act_of(c.kind);
        if (act && same_range(c.u.unary.input, mm.output) && c.u.unary.element_count == count && c.u.unary.dtype == mm.dtype) {
            HoloKernelCall f;
            memset(&f, 0, sizeof f);
            f.kind = HOLO_K_MATMUL_ACTIVATION;
            f.u.matmul_activation.mm = mm;
            f.u.matmul_activation.mm.output = c.u.unary.output;
            f.u.matmul_activation.act = act;
            c = f;
            dead[i] = true;
            ++fused;
        } else if (c.kind == HOLO_K_ADD && c.u.binary.element_count == count && c.u.binary.dtype == mm.dtype &&
                   (same_range(c.u.binary.a, mm.output) != same_range(c.u.binary.b, mm.output))) {
            HoloKernelCall f;
            memset(&f, 0, sizeof f);
            f.kind = HOLO_K_MATMUL_ADD;
            f.u.matmul_add.mm = mm;
            f.u.matmul_add.mm.output = c.u.binary.output;
            f.u.matmul_add.residual = same_range(c.u.binary.a, mm.output) ? c.u.binary.b : c.u.binary.a;
            c = f;
            dead[i] = true;
            ++fused;
        }
    }
    std::vector<HoloKernelCall> kept;
    for (size_t i = 0; i < calls.size(); ++i)
        if (!dead[i]) kept.push_back(calls[i]);
    calls.swap(kept);
    return fused;
}

int32_t run_calls(holo_b200_session* s) {
    for (const HoloKernelCall& c : s->calls) HOLO_TRY(holo_dispatch_internal(s->ctx, &c, s->ws));
    return HOLO_OK;
}

}  // namespace

extern "C" int32_t holo_b200_session_load(holo_b200_ctx* ctx, const uint8_t* archive, uint64_t len, int32_t verify,
                                          holo_b200_session** out) {
    if (!ctx || !archive || !out) return holo_fail(HOLO_ERR_INIT, "backend init failed: null argument");
    HOLO_CUDA(cudaSetDevice(ctx->device));
    holo_b200_session* s = new holo_b200_session();
    s->ctx = ctx;
    int32_t rc = holo_archive_parse(archive, len, verify != 0, &s->ar);
    if (rc != HOLO_OK) {
        delete s;
        return rc;
    }
    // execution order: ExecPlan levels, else one level in call order (session.rs:473)
    if (s->ar.exec_plan.empty()) {
        s->calls = s->ar.calls;
    } else {
        for (const auto& lv : s->ar.exec_plan)
            for (uint32_t idx : lv) s->calls.push_back(s->ar.calls[idx]);
    }
    std::set<uint32_t> in_slots, out_slots;
    for (const HoloPort& p : s->ar.inputs) in_slots.insert(p.slot);
    for (const HoloPort& p : s->ar.outputs) out_slots.insert(p.slot);
    s->fused = fuse_matmul_epilogue(s->calls, out_slots);

    // slot sizing (session.rs:544-629)
    uint32_t n_slots = 0;
    auto bump = [&](uint32_t slot) {
        if (slot != HOLO_NO_SLOT && slot + 1 > n_slots) n_slots = slot + 1;
    };
    for (HoloKernelCall& c : s->calls) {
        HoloRefList refs;
        if (holo_collect_refs(&c, &refs))
            for (int r = 0; r < refs.n; ++r) bump(refs.refs[r]->slot);
    }
    for (const HoloPort& p : s->ar.inputs) bump(p.slot);
    for (const HoloPort& p : s->ar.outputs) bump(p.slot);
    for (const HoloConstant& k : s->ar.constants) bump(k.slot);
    std::vector<uint64_t> need(n_slots, 0);
    for (HoloKernelCall& c : s->calls) {
        HoloRefList refs;
        if (!holo_collect_refs(&c, &refs)) continue;
        for (int r = 0; r < refs.n; ++r) {
            const HoloBufferRef& b = *refs.refs[r];
            if (b.slot == HOLO_NO_SLOT) continue;
            uint64_t ext = b.offset + (b.length ? b.length : refs.out_bytes[r]);
            need[b.slot] = std::max(need[b.slot], ext);
        }
    }
    for (const HoloPort& p : s->ar.inputs) need[p.slot] = std::max(need[p.slot], p.element_count * holo_dtype_size(p.dtype));
    for (const HoloPort& p : s->ar.outputs) need[p.slot] = std::max(need[p.slot], p.element_count * holo_dtype_size(p.dtype));
    for (const HoloConstant& k : s->ar.constants) need[k.slot] = std::max(need[k.slot], k.len);

    // in-place KV move: the output port of a KvCacheWrite shares its cache's buffer
    std::vector<int64_t> alias(n_slots, -1);
    for (const HoloKernelCall& c : s->calls) {
        if (c.kind != HOLO_K_KV_CACHE_WRITE) continue;
        const HoloKvCacheWriteCall& k = c.u.kv_cache_write;
        if (in_slots.count(k.cache.slot) && out_slots.count(k.output.slot) && k.cache.offset == 0 && k.output.offset == 0 &&
            k.cache.slot != k.output.slot) {
            alias[k.output.slot] = k.cache.slot;
            need[k.cache.slot] = std::max(need[k.cache.slot], need[k.output.slot]);
            ++s->moved_in_place;
        }
    }
    rc = holo_b200_workspace_create(ctx, n_slots, &s->ws);
    for (uint32_t i = 0; rc == HOLO_OK && i < n_slots; ++i) {
        if (alias[i] >= 0) continue;
        uint64_t bytes = std::max<uint64_t>(need[i], 64);
        bytes = (bytes + 63) & ~63ull;
        rc = holo_b200_workspace_alloc(s->ws, i, bytes);
        s->device_bytes += bytes;
    }
    for (uint32_t i = 0; rc == HOLO_OK && i < n_slots; ++i) {
        if (alias[i] < 0) continue;
        void* p;
        uint64_t nb;
        rc = holo_b200_workspace_slot(s->ws, (uint32_t)alias[i], &p, &nb);
        if (rc == HOLO_OK) rc = holo_b200_workspace_bind(s->ws, i, p, nb);
    }
    for (size_t i = 0; rc == HOLO_OK && i < s->ar.constants.size(); ++i) {
        const HoloConstant& k = s->ar.constants[i];
        HoloBufferRef ref = {k.slot, 0, 0};
        rc = holo_b200_workspace_upload(s->ws, ref, k.bytes, k.len);
    }
    if (rc == HOLO_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = holo_fail(HOLO_ERR_INIT, "backend init failed: constant upload");
    if (rc != HOLO_OK) {
        if (s->ws) holo_b200_workspace_destroy(s->ws);
        delete s;
        return rc;
    }
    *out = s;
    return HOLO_OK;
}

extern "C" void holo_b200_session_destroy(holo_b200_session* s) {
    if (!s) return;
    cudaSetDevice(s->ctx->device);
    cudaStreamSynchronize(s->ctx->stream);
    if (s->graph) cudaGraphExecDestroy(s->graph);
    if (s->ws) holo_b200_workspace_destroy(s->ws);
    delete s;
}

extern "C" holo_b200_workspace* holo_b200_session_workspace(holo_b200_session* s) { return s ? s->ws : nullptr; }

extern "C" int32_t holo_b200_session_info(holo_b200_session* s, uint32_t* n_calls, uint32_t* n_fused, uint32_t* n_moved,
                                          uint32_t* n_inputs, uint32_t* n_outputs, uint64_t* device_bytes) {
    if (!s) return holo_fail(HOLO_ERR_INIT, "null session");
    if (n_calls) *n_calls = (uint32_t)s->calls.size();
    if (n_fused) *n_fused = s->fused;
    if (n_moved) *n_moved = s->moved_in_place;
    if (n_inputs) *n_inputs = (uint32_t)s->ar.inputs.size();
    if (n_outputs) *n_outputs = (uint32_t)s->ar.outputs.size();
    if (device_bytes) *device_bytes = s->device_bytes;
    return HOLO_OK;
}

extern "C" int32_t holo_b200_session_port(holo_b200_session* s, int32_t is_output, uint32_t index, char* name, uint32_t name_cap,
                                          uint32_t* slot, uint64_t* element_count, uint8_t* dtype) {
    if (!s) return holo_fail(HOLO_ERR_INIT, "null session");
    const std::vector<HoloPort>& ports = is_output ? s->ar.outputs : s->ar.inputs;
    if (index >= ports.size()) return holo_fail(HOLO_ERR_SHAPE_MISMATCH, "shape mismatch: port index %u of %zu", index, ports.size());
    const HoloPort& p = ports[index];
    if (name && name_cap) {
        size_t n = std::min<size_t>(p.name.size(), name_cap - 1);
        memcpy(name, p.name.data(), n);
        name[n] = 0;
    }
    if (slot) *slot = p.slot;
    if (element_count) *element_count = p.element_count;
    if (dtype) *dtype = p.dtype;
    return HOLO_OK;
}

// Copy of call `index` of the post-fusion execution order (for inspection and tests).
extern "C" int32_t holo_b200_session_call(holo_b200_session* s, uint32_t index, HoloKernelCall* out) {
    if (!s || !out) return holo_fail(HOLO_ERR_INIT, "null argument");
    if (index >= s->calls.size()) return holo_fail(HOLO_ERR_SHAPE_MISMATCH, "shape mismatch: call index %u of %zu", index, s->calls.size());
    *out = s->calls[index];
    return HOLO_OK;
}

extern "C" int32_t holo_b200_session_execute(holo_b200_session* s) {
    if (!s) return holo_fail(HOLO_ERR_INIT, "null session");
    HOLO_CUDA(cudaSetDevice(s->ctx->device));
    if (s->graph) {
        HOLO_CUDA(cudaGraphLaunch(s->graph, s->ctx->stream));
        s->ctx->launches += s->calls.size();
        return HOLO_OK;
    }
    return run_calls(s);
}

// Capture one walk into a CUDA graph; later executes replay it. Run at least one eager
// execute first so that scratch buffers and LUT tables already exist (allocation is not
// allowed while a stream is capturing).
extern "C" int32_t holo_b200_session_capture(holo_b200_session* s) {
    if (!s) return holo_fail(HOLO_ERR_INIT, "null session");
    HOLO_CUDA(cudaSetDevice(s->ctx->device));
    if (s->graph) {
        cudaGraphExecDestroy(s->graph);
        s->graph = nullptr;
    }
    HOLO_CUDA(cudaStreamSynchronize(s->ctx->stream));
    HOLO_CUDA(cudaStreamBeginCapture(s->ctx->stream, cudaStreamCaptureModeThreadLocal));
    int32_t rc = run_calls(s);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(s->ctx->stream, &g);
    if (rc != HOLO_OK) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (e != cudaSuccess) return holo_cuda_fail(e, "cudaStreamEndCapture");
    e = cudaGraphInstantiate(&s->graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return holo_cuda_fail(e, "cudaGraphInstantiate");
    return HOLO_OK;
}

// Parse (and optionally verify) an archive image without touching a device: the HoloLoader
// checks of crates/hologram-archive/src/loader.rs:141-267.
extern "C" int32_t holo_b200_archive_check(const uint8_t* archive, uint64_t len, int32_t verify, uint32_t* n_calls,
                                           uint32_t* n_inputs, uint32_t* n_outputs, uint32_t* n_constants) {
    if (!archive) return holo_fail(HOLO_ERR_INIT, "backend init failed: null archive");
    HoloArchive ar;
    HOLO_TRY(holo_archive_parse(archive, len, verify != 0, &ar));
    if (n_calls) *n_calls = (uint32_t)ar.calls.size();
    if (n_inputs) *n_inputs = (uint32_t)ar.inputs.size();
    if (n_outputs) *n_outputs = (uint32_t)ar.outputs.size();
    if (n_constants) *n_constants = (uint32_t)ar.constants.size();
    return HOLO_OK;
}
