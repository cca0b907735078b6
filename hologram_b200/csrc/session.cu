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

// A merged group of sibling matmuls: products of one A against several constant weights,
// executed as one matmul against the column-concatenated weights with one output segment each.
struct MergedMatmul {
    HoloBufferRef a;
    uint32_t m = 0, k = 0, n = 0, nseg = 0;
    void* b_concat = nullptr;          // [k, n] bf16, owned by the session
    HoloBufferRef out[3];
    uint32_t width[3] = {0, 0, 0};
    uint8_t act[3] = {0, 0, 0};
    HoloBufferRef b_src[3];
};

// A run of mutually independent small glue calls executed as one launch.
struct MicroBatch {
    HoloMicroOp* dev_ops = nullptr;    // owned by the session
    uint32_t nops = 0, total_ctas = 0, ncalls = 0;
};

struct SessionNode {
    int merged = -1;                   // index into holo_b200_session::merged, or -1
    int batch = -1;                    // index into holo_b200_session::batches, or -1
    HoloKernelCall call;               // the plain call when both are -1
    // AllReduce followed by the residual Add, run as one launch: `call` is the AllReduce,
    // `residual` / `sum_out` come from the Add
    bool reduce_add = false;
    HoloBufferRef residual = {HOLO_NO_SLOT, 0, 0}, sum_out = {HOLO_NO_SLOT, 0, 0};
};

struct holo_b200_session {
    holo_b200_ctx* ctx = nullptr;
    holo_b200_workspace* ws = nullptr;
    HoloArchive ar;
    std::vector<HoloKernelCall> calls;  // execution order, after fusion (merged groups keep their members here)
    std::vector<SessionNode> nodes;     // what a walk actually launches
    std::vector<MergedMatmul> merged;
    std::vector<MicroBatch> batches;
    uint32_t fused = 0, moved_in_place = 0, merged_calls = 0, batched_calls = 0, reduce_adds = 0;
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

bool is_plain_or_act_matmul(const HoloKernelCall& c) { return c.kind == HOLO_K_MATMUL || c.kind == HOLO_K_MATMUL_ACTIVATION; }

// Sibling-matmul merge (a device-side analogue of the reference's load-time weight-layout
// choices, e.g. panel packing, crates/hologram-compute/src/layout.rs): consecutive MatMul /
// MatMulActivation calls that multiply the same A by constant weights become one product
// against the column-concatenated weights, each member keeping its own output buffer and
// epilogue. Per-element arithmetic is unchanged (same k-order accumulation per column).
void plan_sibling_merges(holo_b200_session* s, const std::set<uint32_t>& const_slots, const std::set<uint32_t>& written_slots) {
    const std::vector<HoloKernelCall>& calls = s->calls;
    size_t i = 0;
    while (i < calls.size()) {
        SessionNode node;
        node.call = calls[i];
        if (!is_plain_or_act_matmul(calls[i])) {
            s->nodes.push_back(node);
            ++i;
            continue;
        }
        const HoloMatMulCall& first = calls[i].u.matmul;
        auto mergeable = [&](const HoloKernelCall& c) {
            if (!is_plain_or_act_matmul(c)) return false;
            const HoloMatMulCall& mm = c.u.matmul;
            return mm.dtype == HOLO_DTYPE_BF16 && !mm.b_packed && mm.a.slot == first.a.slot && mm.a.offset == first.a.offset &&
                   mm.m == first.m && mm.k == first.k && (mm.n % 32) == 0 && (mm.k % 8) == 0 && const_slots.count(mm.b.slot) &&
                   !written_slots.count(mm.b.slot) && mm.b.offset % 16 == 0 && (uint64_t)mm.m * mm.n * mm.k >= (1ull << 18);
        };
        size_t j = i;
        MergedMatmul g;
        while (j < calls.size() && g.nseg < 3 && mergeable(calls[j])) {
            const HoloMatMulCall& mm = calls[j].u.matmul;
            bool distinct = true;
            for (uint32_t t = 0; t < g.nseg; ++t) distinct &= g.out[t].slot != mm.output.slot;
            if (!distinct || mm.output.slot == first.a.slot) break;
            g.out[g.nseg] = mm.output;
            g.b_src[g.nseg] = mm.b;
            g.width[g.nseg] = mm.n;
            g.act[g.nseg] = calls[j].kind == HOLO_K_MATMUL_ACTIVATION ? calls[j].u.matmul_activation.act : 0;
            g.n += mm.n;
            ++g.nseg;
            ++j;
        }
        if (g.nseg >= 2 && first.m <= 128 && !getenv("HOLO_SESSION_NO_MERGE")) {
            g.a = first.a;
            g.m = first.m;
            g.k = first.k;
            node.merged = (int)s->merged.size();
            s->merged.push_back(g);
            s->nodes.push_back(node);
            s->merged_calls += g.nseg;
            i = j;
        } else {
            s->nodes.push_back(node);
            ++i;
        }
    }
}

int32_t build_merged_weights(holo_b200_session* s) {
    for (MergedMatmul& g : s->merged) {
        HOLO_CUDA(cudaMalloc(&g.b_concat, (size_t)g.k * g.n * 2));
        s->device_bytes += (uint64_t)g.k * g.n * 2;
        uint32_t col = 0;
        for (uint32_t t = 0; t < g.nseg; ++t) {
            uint8_t* src;
            HOLO_TRY(holo_resolve(s->ws, g.b_src[t], (uint64_t)g.k * g.width[t] * 2, &src, nullptr));
            HOLO_CUDA(cudaMemcpy2DAsync((uint8_t*)g.b_concat + (size_t)col * 2, (size_t)g.n * 2, src, (size_t)g.width[t] * 2,
                                        (size_t)g.width[t] * 2, g.k, cudaMemcpyDeviceToDevice, s->ctx->stream));
            col += g.width[t];
        }
    }
    HOLO_CUDA(cudaStreamSynchronize(s->ctx->stream));
    // the separate weights are no longer read by any node: give their memory back
    std::set<uint32_t> still_used;
    for (const SessionNode& n : s->nodes) {
        if (n.merged >= 0) continue;
        HoloKernelCall tmp = n.call;
        HoloRefList refs;
        if (holo_collect_refs(&tmp, &refs))
            for (int r = 0; r < refs.n; ++r) still_used.insert(refs.refs[r]->slot);
    }
    for (const MergedMatmul& g : s->merged)
        for (uint32_t t = 0; t < g.nseg; ++t)
            if (!still_used.count(g.b_src[t].slot)) {
                uint64_t nb = 0;
                void* ptr = nullptr;
                if (holo_b200_workspace_slot(s->ws, g.b_src[t].slot, &ptr, &nb) == HOLO_OK) s->device_bytes -= std::min<uint64_t>(s->device_bytes, nb);
                holo_b200_workspace_bind(s->ws, g.b_src[t].slot, nullptr, 0);
            }
    return HOLO_OK;
}

int32_t run_merged(holo_b200_session* s, const MergedMatmul& g) {
    uint8_t* a;
    HOLO_TRY(holo_resolve(s->ws, g.a, (uint64_t)g.m * g.k * 2, &a, nullptr));
    HoloMatmulSeg segs[3];
    for (uint32_t t = 0; t < g.nseg; ++t) {
        uint8_t* o;
        HOLO_TRY(holo_resolve(s->ws, g.out[t], (uint64_t)g.m * g.width[t] * 2, &o, nullptr));
        segs[t].out = o;
        segs[t].residual = nullptr;
        segs[t].width = g.width[t];
        segs[t].fused_act = g.act[t];
    }
    return holo_launch_matmul_multi(s->ctx, a, g.b_concat, g.m, g.k, g.n, HOLO_DTYPE_BF16, segs, g.nseg);
}

// Tensor parallel: an AllReduce over a buffer, directly followed by the Add of that buffer and
// a residual, with nothing else reading the reduced buffer afterwards, becomes one node (one
// launch of the peer-memory kernel: sum over ranks, truncate, add the residual, truncate).
void fuse_all_reduce_add(holo_b200_session* s, const std::set<uint32_t>& output_slots) {
    std::vector<SessionNode> out;
    for (size_t i = 0; i < s->nodes.size(); ++i) {
        SessionNode n = s->nodes[i];
        const bool plain = n.merged < 0 && n.batch < 0;
        if (plain && n.call.kind == HOLO_K_ALL_REDUCE && i + 1 < s->nodes.size()) {
            const SessionNode& nx = s->nodes[i + 1];
            const HoloAllReduceCall& ar = n.call.u.all_reduce;
            if (nx.merged < 0 && nx.batch < 0 && nx.call.kind == HOLO_K_ADD && nx.call.u.binary.element_count == ar.element_count &&
                nx.call.u.binary.dtype == ar.dtype && !output_slots.count(ar.buffer.slot) &&
                (same_range(nx.call.u.binary.a, ar.buffer) != same_range(nx.call.u.binary.b, ar.buffer))) {
                bool read_later = false;
                for (size_t j = i + 2; j < s->nodes.size() && !read_later; ++j) {
                    if (s->nodes[j].merged >= 0) {
                        read_later = s->merged[s->nodes[j].merged].a.slot == ar.buffer.slot;
                        continue;
                    }
                    HoloKernelCall tmp = s->nodes[j].call;
                    HoloRefList refs;
                    if (!holo_collect_refs(&tmp, &refs)) continue;
                    for (int r = 0; r < refs.n; ++r)
                        if (refs.refs[r]->slot == ar.buffer.slot && !refs.written[r]) read_later = true;
                }
                if (!read_later) {
                    n.reduce_add = true;
                    n.residual = same_range(nx.call.u.binary.a, ar.buffer) ? nx.call.u.binary.b : nx.call.u.binary.a;
                    n.sum_out = nx.call.u.binary.output;
                    out.push_back(n);
                    ++s->reduce_adds;
                    ++i;  // the Add is absorbed
                    continue;
                }
            }
        }
        out.push_back(n);
    }
    s->nodes.swap(out);
}

int32_t run_reduce_add(holo_b200_session* s, const SessionNode& n) {
    const HoloAllReduceCall& ar = n.call.u.all_reduce;
    const uint64_t bytes = ar.element_count * holo_dtype_size(ar.dtype);
    uint8_t *buf, *res, *dst;
    HOLO_TRY(holo_resolve(s->ws, ar.buffer, bytes, &buf, nullptr));
    HOLO_TRY(holo_resolve(s->ws, n.residual, bytes, &res, nullptr));
    HOLO_TRY(holo_resolve(s->ws, n.sum_out, bytes, &dst, nullptr));
    return holo_all_reduce_add(s->ctx, buf, res, dst, ar.element_count, ar.dtype);
}

bool batchable_kind(uint16_t k) {
    return k == HOLO_K_KV_CACHE_WRITE || k == HOLO_K_ROTARY || k == HOLO_K_QUANTIZE_ROWS_I8 || k == HOLO_K_ADD || k == HOLO_K_MUL;
}

// Group consecutive, mutually independent small glue calls (no member reads or writes a slot
// another member writes) into single launches. Each member is first dispatched in recording
// mode, which runs its full validation and slot resolution but appends a descriptor instead
// of launching; slots never move after load, so the descriptors stay valid for every walk.
int32_t plan_micro_batches(holo_b200_session* s) {
    if (getenv("HOLO_SESSION_NO_BATCH")) return HOLO_OK;
    std::vector<SessionNode> out;
    size_t i = 0;
    while (i < s->nodes.size()) {
        const SessionNode& n0 = s->nodes[i];
        if (n0.merged >= 0 || !batchable_kind(n0.call.kind)) {
            out.push_back(n0);
            ++i;
            continue;
        }
        std::set<uint32_t> reads, writes;
        size_t j = i;
        while (j < s->nodes.size() && j - i < 64) {
            const SessionNode& nj = s->nodes[j];
            if (nj.merged >= 0 || !batchable_kind(nj.call.kind)) break;
            HoloKernelCall tmp = nj.call;
            HoloRefList refs;
            if (!holo_collect_refs(&tmp, &refs)) break;
            bool ok = true;
            for (int r = 0; r < refs.n && ok; ++r) {
                const uint32_t slot = refs.refs[r]->slot;
                if (slot == HOLO_NO_SLOT) continue;
                // aliased slots (the in-place KV move) share memory: compare device pointers
                void* ptr = nullptr;
                uint64_t nb = 0;
                if (holo_b200_workspace_slot(s->ws, slot, &ptr, &nb) != HOLO_OK) { ok = false; break; }
                const uint32_t key = (uint32_t)((uintptr_t)ptr >> 6);
                if (refs.written[r]) ok = !reads.count(key) && !writes.count(key);
                else ok = !writes.count(key);
            }
            if (!ok) break;
            for (int r = 0; r < refs.n; ++r) {
                const uint32_t slot = refs.refs[r]->slot;
                if (slot == HOLO_NO_SLOT) continue;
                void* ptr = nullptr;
                uint64_t nb = 0;
                holo_b200_workspace_slot(s->ws, slot, &ptr, &nb);
                const uint32_t key = (uint32_t)((uintptr_t)ptr >> 6);
                // a KvCacheWrite reads its cache only to carry it over: in place that is no access
                if (nj.call.kind == HOLO_K_KV_CACHE_WRITE && refs.refs[r] == &tmp.u.kv_cache_write.cache) continue;
                (refs.written[r] ? writes : reads).insert(key);
            }
            ++j;
        }
        if (j - i < 2) {
            out.push_back(n0);
            ++i;
            continue;
        }
        std::vector<HoloMicroOp> ops;
        s->ctx->record = &ops;
        s->ctx->record_failed = false;
        int32_t rc = HOLO_OK;
        for (size_t t = i; t < j && rc == HOLO_OK; ++t) rc = holo_dispatch_internal(s->ctx, &s->nodes[t].call, s->ws);
        s->ctx->record = nullptr;
        if (rc != HOLO_OK) return rc;
        if (s->ctx->record_failed || ops.size() != j - i) {   // something in the run cannot be batched: keep the calls
            for (size_t t = i; t < j; ++t) out.push_back(s->nodes[t]);
            i = j;
            continue;
        }
        MicroBatch b;
        uint32_t cta = 0;
        for (HoloMicroOp& op : ops) {
            op.cta_begin = cta;
            cta += op.cta_count;
        }
        b.nops = (uint32_t)ops.size();
        b.total_ctas = cta;
        b.ncalls = (uint32_t)(j - i);
        HOLO_CUDA(cudaMalloc(&b.dev_ops, ops.size() * sizeof(HoloMicroOp)));
        HOLO_CUDA(cudaMemcpy(b.dev_ops, ops.data(), ops.size() * sizeof(HoloMicroOp), cudaMemcpyHostToDevice));
        SessionNode node;
        node.batch = (int)s->batches.size();
        node.call = n0.call;
        s->batches.push_back(b);
        s->batched_calls += b.ncalls;
        out.push_back(node);
        i = j;
    }
    s->nodes.swap(out);
    return HOLO_OK;
}

int32_t run_calls(holo_b200_session* s) {
    for (const SessionNode& n : s->nodes) {
        if (n.reduce_add) HOLO_TRY(run_reduce_add(s, n));
        else if (n.merged >= 0) HOLO_TRY(run_merged(s, s->merged[n.merged]));
        else if (n.batch >= 0) HOLO_TRY(holo_launch_micro_batch(s->ctx, s->batches[n.batch].dev_ops, s->batches[n.batch].nops, s->batches[n.batch].total_ctas));
        else HOLO_TRY(holo_dispatch_internal(s->ctx, &n.call, s->ws));
    }
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
    {
        std::set<uint32_t> const_slots, written_slots;
        for (const HoloConstant& k : s->ar.constants) const_slots.insert(k.slot);
        for (HoloKernelCall& c : s->calls) {
            HoloRefList refs;
            if (holo_collect_refs(&c, &refs))
                for (int r = 0; r < refs.n; ++r)
                    if (refs.written[r]) written_slots.insert(refs.refs[r]->slot);
        }
        for (const HoloPort& p : s->ar.inputs) written_slots.insert(p.slot);   // inputs are rewritten by the caller
        plan_sibling_merges(s, const_slots, written_slots);
        fuse_all_reduce_add(s, out_slots);
    }

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
    if (rc == HOLO_OK) rc = build_merged_weights(s);
    if (rc == HOLO_OK) rc = plan_micro_batches(s);
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
    for (MergedMatmul& g : s->merged)
        if (g.b_concat) cudaFree(g.b_concat);
    for (MicroBatch& b : s->batches)
        if (b.dev_ops) cudaFree(b.dev_ops);
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

extern "C" int32_t holo_b200_session_nodes(holo_b200_session* s, uint32_t* n_nodes, uint32_t* n_merged_calls) {
    if (!s) return holo_fail(HOLO_ERR_INIT, "null session");
    if (n_nodes) *n_nodes = (uint32_t)s->nodes.size();
    if (n_merged_calls) *n_merged_calls = s->merged_calls + s->batched_calls + 2 * s->reduce_adds;
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
        s->ctx->launches += s->nodes.size();
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
