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

#include <array>
#include <string>
#include <unordered_map>

#include "session.h"

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

// fuse_matmul_epilogue (session.rs:2150-2377), with the reference's rules: the producer is a MatMul whose
// output slot has exactly one producer and exactly one reader in the whole call list and is not a graph
// output; the reader is a table-backed activation over it, or an Add with it as one operand whose other
// operand (the residual) is produced at a strictly earlier schedule level than the matmul (or by no call:
// an input or a constant). The fused call takes the PRODUCER's place; the reader is dropped. For f32 an
// activation that is the single reader of the Add's result is absorbed too (MatMulAddActivation: with no
// narrowing to skip, the triple is bit-identical to the three calls).
uint32_t fuse_matmul_epilogue(std::vector<HoloKernelCall>& calls, std::vector<uint32_t>& level, const std::set<uint32_t>& output_slots) {
    const size_t n = calls.size();
    std::unordered_map<uint32_t, uint32_t> prod_count, read_count, slot_level;
    std::unordered_map<uint32_t, size_t> read_idx;
    for (size_t i = 0; i < n; ++i) {
        HoloKernelCall tmp = calls[i];
        HoloRefList refs;
        if (!holo_collect_refs(&tmp, &refs)) continue;
        for (int r = 0; r < refs.n; ++r) {
            const uint32_t slot = refs.refs[r]->slot;
            if (slot == HOLO_NO_SLOT) continue;
            if (refs.written[r]) {
                ++prod_count[slot];
                slot_level[slot] = level[i];
                if (calls[i].kind == HOLO_K_ALL_REDUCE) {   // rewritten in place: also a reader
                    ++read_count[slot];
                    read_idx[slot] = i;
                }
            } else {
                ++read_count[slot];
                read_idx[slot] = i;
            }
        }
    }
    std::vector<bool> absorbed(n, false), has_fused(n, false);
    std::vector<HoloKernelCall> fused(n);
    uint32_t count = 0;
    for (size_t i = 0; i < n; ++i) {
        if (calls[i].kind != HOLO_K_MATMUL) continue;
        const HoloMatMulCall mm = calls[i].u.matmul;
        if (mm.dtype != HOLO_DTYPE_BF16 && mm.dtype != HOLO_DTYPE_F16 && mm.dtype != HOLO_DTYPE_F32) continue;
        const uint32_t s = mm.output.slot;
        if (s == HOLO_NO_SLOT || output_slots.count(s)) continue;
        if (prod_count[s] != 1 || read_count[s] != 1) continue;
        const size_t j = read_idx[s];
        if (j == i || absorbed[j]) continue;
        const HoloKernelCall& c = calls[j];
        const uint64_t cells = (uint64_t)mm.m * mm.n;
        const uint8_t act = fused_act_of(c.kind);
        HoloKernelCall f;
        memset(&f, 0, sizeof f);
        if (act) {
            if (!same_range(c.u.unary.input, mm.output) || c.u.unary.element_count != cells || c.u.unary.dtype != mm.dtype) continue;
            f.kind = HOLO_K_MATMUL_ACTIVATION;
            f.u.matmul_activation.mm = mm;
            f.u.matmul_activation.mm.output = c.u.unary.output;
            f.u.matmul_activation.act = act;
            fused[i] = f;
            has_fused[i] = true;
            absorbed[j] = true;
            ++count;
        } else if (c.kind == HOLO_K_ADD) {
            if (c.u.binary.element_count != cells || c.u.binary.dtype != mm.dtype) continue;
            if (same_range(c.u.binary.a, mm.output) == same_range(c.u.binary.b, mm.output)) continue;
            const HoloBufferRef residual = same_range(c.u.binary.a, mm.output) ? c.u.binary.b : c.u.binary.a;
            // the residual must be ready no later than the matmul that absorbs it
            auto rl = slot_level.find(residual.slot);
            if (rl != slot_level.end() && !(rl->second < level[i])) continue;
            const uint32_t add_out = c.u.binary.output.slot;
            bool triple = false;
            if (mm.dtype == HOLO_DTYPE_F32 && add_out != HOLO_NO_SLOT && !output_slots.count(add_out) && prod_count[add_out] == 1 &&
                read_count[add_out] == 1) {
                const size_t k = read_idx[add_out];
                const uint8_t act2 = k != j && !absorbed[k] ? fused_act_of(calls[k].kind) : 0;
                if (act2 && same_range(calls[k].u.unary.input, c.u.binary.output) && calls[k].u.unary.element_count == cells &&
                    calls[k].u.unary.dtype == mm.dtype) {
                    f.kind = HOLO_K_MATMUL_ADD_ACTIVATION;
                    f.u.matmul_add_activation.mm = mm;
                    f.u.matmul_add_activation.mm.output = calls[k].u.unary.output;
                    f.u.matmul_add_activation.residual = residual;
                    f.u.matmul_add_activation.act = act2;
                    absorbed[k] = true;
                    ++count;
                    triple = true;
                }
            }
            if (!triple) {
                f.kind = HOLO_K_MATMUL_ADD;
                f.u.matmul_add.mm = mm;
                f.u.matmul_add.mm.output = c.u.binary.output;
                f.u.matmul_add.residual = residual;
            }
            fused[i] = f;
            has_fused[i] = true;
            absorbed[j] = true;
            ++count;
        }
    }
    std::vector<HoloKernelCall> kept;
    std::vector<uint32_t> kept_level;
    for (size_t i = 0; i < n; ++i) {
        if (absorbed[i]) continue;
        kept.push_back(has_fused[i] ? fused[i] : calls[i]);
        kept_level.push_back(level[i]);
    }
    calls.swap(kept);
    level.swap(kept_level);
    return count;
}

// A RotaryEmbedding whose output is read by a QuantizeRowsI8 over rows of the RoPE's head_dim (the K
// path of a decoder layer) becomes one call that does both; the quantizer then no longer depends on
// a separate launch and can share a batched launch with its siblings. The RoPE output is still
// written (other readers keep working).
uint32_t fuse_rope_quantize(std::vector<HoloKernelCall>& calls, std::vector<uint32_t>& level) {
    if (getenv("HOLO_SESSION_NO_ROPE_QUANT")) return 0;
    uint32_t fused = 0;
    std::vector<bool> dead(calls.size(), false);
    for (size_t i = 0; i < calls.size(); ++i) {
        if (calls[i].kind != HOLO_K_ROTARY) continue;
        const HoloRoPECall ro = calls[i].u.rope;
        for (size_t j = i + 1; j < calls.size() && j < i + 8; ++j) {
            if (dead[j]) continue;
            // stop at anything that rewrites the RoPE's operands or output
            HoloKernelCall tmp = calls[j];
            HoloRefList refs;
            bool clobber = false;
            if (holo_collect_refs(&tmp, &refs))
                for (int r = 0; r < refs.n; ++r)
                    if (refs.written[r] && (refs.refs[r]->slot == ro.output.slot || refs.refs[r]->slot == ro.x.slot ||
                                            refs.refs[r]->slot == ro.cos.slot || refs.refs[r]->slot == ro.sin.slot))
                        clobber = true;
            if (calls[j].kind == HOLO_K_QUANTIZE_ROWS_I8) {
                const HoloQuantizeRowsI8Call q = calls[j].u.quantize_rows_i8;
                // the quantizer moves up to the RoPE's position: nothing in between may touch its outputs
                bool free_to_move = true;
                for (size_t t = i + 1; t < j && free_to_move; ++t) {
                    if (dead[t]) continue;
                    HoloKernelCall mid = calls[t];
                    HoloRefList mr;
                    if (!holo_collect_refs(&mid, &mr)) { free_to_move = false; break; }
                    for (int r = 0; r < mr.n; ++r)
                        if (mr.refs[r]->slot == q.codes.slot || mr.refs[r]->slot == q.scales.slot) free_to_move = false;
                }
                if (free_to_move && same_range(q.input, ro.output) && q.row_len == ro.head_dim && q.rows * q.row_len == ro.element_count &&
                    q.dtype == ro.dtype) {
                    HoloKernelCall f;
                    memset(&f, 0, sizeof f);
                    f.kind = HOLO_K_ROPE_QUANTIZE_ROWS_I8;
                    f.u.rope_quantize.x = ro.x;
                    f.u.rope_quantize.cos = ro.cos;
                    f.u.rope_quantize.sin = ro.sin;
                    f.u.rope_quantize.rope_output = ro.output;
                    f.u.rope_quantize.codes = q.codes;
                    f.u.rope_quantize.scales = q.scales;
                    f.u.rope_quantize.rows = q.rows;
                    f.u.rope_quantize.row_len = q.row_len;
                    f.u.rope_quantize.dtype = q.dtype;
                    calls[i] = f;      // at the RoPE's position: its operands are ready there
                    dead[j] = true;
                    ++fused;
                    break;
                }
            }
            if (clobber) break;
        }
    }
    std::vector<HoloKernelCall> kept;
    std::vector<uint32_t> kept_level;
    for (size_t i = 0; i < calls.size(); ++i)
        if (!dead[i]) {
            kept.push_back(calls[i]);
            kept_level.push_back(level[i]);
        }
    calls.swap(kept);
    level.swap(kept_level);
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
            if (g.gated) {
                // block j of weight t (64 columns) lands at columns 128 j + 64 t of the concatenation
                for (uint32_t j = 0; j < g.width[t] / 64; ++j)
                    HOLO_CUDA(cudaMemcpy2DAsync((uint8_t*)g.b_concat + ((size_t)128 * j + 64 * t) * 2, (size_t)g.n * 2, src + (size_t)64 * j * 2,
                                                (size_t)g.width[t] * 2, 64 * 2, g.k, cudaMemcpyDeviceToDevice, s->ctx->stream));
                continue;
            }
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

int32_t resolve_head_op(holo_b200_session* s, const MergedMatmul& g, uint32_t t, HoloMatmulSeg* seg) {
    seg->head_op = g.head_op[t];
    if (!g.head_op[t]) return HOLO_OK;
    const uint64_t count = (uint64_t)g.m * g.width[t];
    uint8_t* ptr;
    if (g.head_op[t] != 3) {
        HOLO_TRY(holo_resolve(s->ws, g.cos[t], count * 2, &ptr, nullptr));
        seg->cos = ptr;
        HOLO_TRY(holo_resolve(s->ws, g.sin[t], count * 2, &ptr, nullptr));
        seg->sin = ptr;
        HOLO_TRY(holo_resolve(s->ws, g.rope_out[t], count * 2, &ptr, nullptr));
        seg->rope_out = ptr;
    }
    if (g.head_op[t] >= 2) {
        HOLO_TRY(holo_resolve(s->ws, g.codes[t], count, &ptr, nullptr));
        seg->codes = (int8_t*)ptr;
        HOLO_TRY(holo_resolve(s->ws, g.scales[t], count / 128 * 4, &ptr, nullptr));
        seg->scales = (float*)ptr;
    }
    return HOLO_OK;
}

int32_t run_merged(holo_b200_session* s, const MergedMatmul& g) {
    uint8_t* a;
    HOLO_TRY(holo_resolve(s->ws, g.a, (uint64_t)g.m * g.k * 2, &a, nullptr));
    HoloMatmulSeg segs[3];
    if (g.gated) {
        uint8_t* o;
        HOLO_TRY(holo_resolve(s->ws, g.gated_out, (uint64_t)g.m * g.width[0] * 2, &o, nullptr));
        segs[0].out = o;
        segs[0].residual = nullptr;
        segs[0].width = g.width[0];
        segs[0].fused_act = g.act[0];
        segs[0].gated = 1;
        segs[0].b_constant = 1;
        return holo_launch_matmul_multi(s->ctx, a, g.b_concat, g.m, g.k, g.n, HOLO_DTYPE_BF16, segs, 1);
    }
    for (uint32_t t = 0; t < g.nseg; ++t) {
        uint8_t* o;
        HOLO_TRY(holo_resolve(s->ws, g.out[t], (uint64_t)g.m * g.width[t] * 2, &o, nullptr));
        segs[t].out = o;
        segs[t].residual = nullptr;
        segs[t].width = g.width[t];
        segs[t].fused_act = g.act[t];
        HOLO_TRY(resolve_head_op(s, g, t, &segs[t]));
    }
    segs[0].b_constant = 1;   // the concatenated weights are the session's own copy
    return holo_launch_matmul_multi(s->ctx, a, g.b_concat, g.m, g.k, g.n, HOLO_DTYPE_BF16, segs, g.nseg);
}

// The per-head calls that directly follow a merged product and read one of its segments (the RoPE of q, the
// RoPE + quantize of k, the quantize of v in a decoder layer) move into the product's epilogue: the warp that
// stores a head's 128 values applies the call's arithmetic to the stored values in registers. The calls'
// results are bit-for-bit those of the separate launches, which disappear.
void fuse_head_ops(holo_b200_session* s) {
    if (getenv("HOLO_SESSION_NO_HEAD_FUSE")) return;
    std::vector<SessionNode> out;
    for (size_t i = 0; i < s->nodes.size(); ++i) {
        out.push_back(s->nodes[i]);
        if (s->nodes[i].merged < 0) continue;
        MergedMatmul& g = s->merged[s->nodes[i].merged];
        if (g.gated || g.m > 128) continue;
        uint32_t absorbed = 0;
        size_t j = i + 1;
        for (; j < s->nodes.size(); ++j) {
            const SessionNode& nx = s->nodes[j];
            if (nx.merged >= 0 || nx.batch >= 0 || nx.reduce_add || nx.matmul_reduce_add) break;
            const HoloKernelCall& c = nx.call;
            HoloBufferRef x, cs = {HOLO_NO_SLOT, 0, 0}, sn = cs, ro = cs, codes = cs, scales = cs;
            uint8_t op = 0, dtype = 0;
            uint32_t row_len = 0;
            uint64_t count = 0;
            if (c.kind == HOLO_K_ROTARY) {
                op = 1; x = c.u.rope.x; cs = c.u.rope.cos; sn = c.u.rope.sin; ro = c.u.rope.output;
                row_len = c.u.rope.head_dim; count = c.u.rope.element_count; dtype = c.u.rope.dtype;
            } else if (c.kind == HOLO_K_ROPE_QUANTIZE_ROWS_I8) {
                const auto& q = c.u.rope_quantize;
                op = 2; x = q.x; cs = q.cos; sn = q.sin; ro = q.rope_output; codes = q.codes; scales = q.scales;
                row_len = q.row_len; count = q.rows * q.row_len; dtype = q.dtype;
            } else if (c.kind == HOLO_K_QUANTIZE_ROWS_I8) {
                const auto& q = c.u.quantize_rows_i8;
                op = 3; x = q.input; codes = q.codes; scales = q.scales;
                row_len = q.row_len; count = q.rows * q.row_len; dtype = q.dtype;
            } else {
                break;
            }
            int t = -1;
            for (uint32_t u = 0; u < g.nseg; ++u)
                if (same_range(x, g.out[u]) && g.head_op[u] == 0) t = (int)u;
            if (t < 0 || row_len != 128 || dtype != HOLO_DTYPE_BF16 || count != (uint64_t)g.m * g.width[t]) break;
            // what the call writes is nothing the product reads or writes
            bool clash = false;
            for (const HoloBufferRef* w : {&ro, &codes, &scales}) {
                if (w->slot == HOLO_NO_SLOT) continue;
                clash |= w->slot == g.a.slot;
                for (uint32_t u = 0; u < g.nseg; ++u) clash |= w->slot == g.out[u].slot || w->slot == g.cos[u].slot || w->slot == g.sin[u].slot;
            }
            // ... and nothing the call itself reads (the separate launches refuse overlapping operands)
            for (const HoloBufferRef* w : {&ro, &codes, &scales})
                for (const HoloBufferRef* r : {&x, &cs, &sn, &ro, &codes, &scales})
                    if (w != r && w->slot != HOLO_NO_SLOT && w->slot == r->slot) clash = true;
            if (clash) break;
            // would the product take it? (resolve the operands as a walk would)
            MergedMatmul trial = g;
            trial.head_op[t] = op;
            trial.cos[t] = cs; trial.sin[t] = sn; trial.rope_out[t] = ro; trial.codes[t] = codes; trial.scales[t] = scales;
            HoloMatmulSeg segs[3];
            bool ok = true;
            for (uint32_t u = 0; u < trial.nseg && ok; ++u) {
                uint8_t* o;
                ok = holo_resolve(s->ws, trial.out[u], (uint64_t)trial.m * trial.width[u] * 2, &o, nullptr) == HOLO_OK;
                segs[u].out = o;
                segs[u].width = trial.width[u];
                segs[u].fused_act = trial.act[u];
                ok = ok && resolve_head_op(s, trial, u, &segs[u]) == HOLO_OK;
            }
            if (!ok || !holo_matmul_head_ops_ok(trial.m, trial.k, trial.n, HOLO_DTYPE_BF16, segs, trial.nseg)) break;
            g = trial;
            ++absorbed;
        }
        s->head_fused += absorbed;
        i = j - 1;   // the absorbed nodes are dropped
    }
    s->nodes.swap(out);
}

// Gated FFN: a merged pair {act(A W0), A W1} whose two results are read only by the Mul that follows
// becomes one product with a gated epilogue; the Mul node is absorbed and the two intermediates are
// never written. Per-element arithmetic is that of the three calls (both factors narrowed before
// the multiply, one narrowing after).
void fuse_gated_pairs(holo_b200_session* s, const std::set<uint32_t>& output_slots) {
    if (getenv("HOLO_SESSION_NO_GATED")) return;
    std::vector<SessionNode> out;
    for (size_t i = 0; i < s->nodes.size(); ++i) {
        SessionNode n = s->nodes[i];
        if (n.merged >= 0 && i + 1 < s->nodes.size()) {
            MergedMatmul& g = s->merged[n.merged];
            const SessionNode& nx = s->nodes[i + 1];
            const uint64_t count = (uint64_t)g.m * g.width[0];
            bool ok = g.nseg == 2 && g.act[0] != 0 && g.act[1] == 0 && g.width[0] == g.width[1] && (g.width[0] % 64) == 0 &&
                      nx.merged < 0 && nx.batch < 0 && nx.call.kind == HOLO_K_MUL && nx.call.u.binary.dtype == HOLO_DTYPE_BF16 &&
                      nx.call.u.binary.element_count == count && !output_slots.count(g.out[0].slot) && !output_slots.count(g.out[1].slot);
            if (ok) {
                const HoloBinaryCall& b = nx.call.u.binary;
                ok = (same_range(b.a, g.out[0]) && same_range(b.b, g.out[1])) || (same_range(b.a, g.out[1]) && same_range(b.b, g.out[0]));
            }
            for (size_t j = i + 2; ok && j < s->nodes.size(); ++j) {   // nobody else reads the two intermediates
                if (s->nodes[j].merged >= 0) {
                    const uint32_t a = s->merged[s->nodes[j].merged].a.slot;
                    ok = a != g.out[0].slot && a != g.out[1].slot;
                    continue;
                }
                HoloKernelCall tmp = s->nodes[j].call;
                HoloRefList refs;
                if (!holo_collect_refs(&tmp, &refs)) continue;
                for (int r = 0; r < refs.n; ++r)
                    if (!refs.written[r] && (refs.refs[r]->slot == g.out[0].slot || refs.refs[r]->slot == g.out[1].slot)) ok = false;
            }
            if (ok) {
                g.gated = true;
                g.gated_out = nx.call.u.binary.output;
                s->merged_calls += 1;
                out.push_back(n);
                ++i;   // the Mul is absorbed
                continue;
            }
        }
        out.push_back(n);
    }
    s->nodes.swap(out);
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

// Tensor parallel: a plain MatMul whose product is only read by the AllReduce + Add node that
// follows becomes one node: the row-parallel projection, the sum over the ranks and the residual
// add in one launch (the exchange runs in the matmul's epilogue over peer memory).
void fuse_matmul_reduce_add(holo_b200_session* s) {
    if (getenv("HOLO_SESSION_NO_MATMUL_AR")) return;
    std::vector<SessionNode> out;
    for (size_t i = 0; i < s->nodes.size(); ++i) {
        SessionNode n = s->nodes[i];
        if (n.merged < 0 && n.batch < 0 && !n.reduce_add && n.call.kind == HOLO_K_MATMUL && i + 1 < s->nodes.size()) {
            const SessionNode& nx = s->nodes[i + 1];
            const HoloMatMulCall& mm = n.call.u.matmul;
            if (nx.reduce_add && mm.dtype == HOLO_DTYPE_BF16 && same_range(nx.call.u.all_reduce.buffer, mm.output) &&
                nx.call.u.all_reduce.element_count == (uint64_t)mm.m * mm.n && nx.call.u.all_reduce.dtype == mm.dtype) {
                n.matmul_reduce_add = true;
                n.residual = nx.residual;
                n.sum_out = nx.sum_out;
                out.push_back(n);
                ++s->reduce_adds;   // one more call absorbed
                ++i;
                continue;
            }
        }
        out.push_back(n);
    }
    s->nodes.swap(out);
}

int32_t run_matmul_reduce_add(holo_b200_session* s, const SessionNode& n) {
    const HoloMatMulCall& mm = n.call.u.matmul;
    const uint64_t ob = (uint64_t)mm.m * mm.n * 2;
    uint8_t *a, *b, *res, *dst;
    HOLO_TRY(holo_resolve(s->ws, mm.a, (uint64_t)mm.m * mm.k * 2, &a, nullptr));
    HOLO_TRY(holo_resolve(s->ws, mm.b, (uint64_t)mm.k * mm.n * 2, &b, nullptr));
    HOLO_TRY(holo_resolve(s->ws, n.residual, ob, &res, nullptr));
    HOLO_TRY(holo_resolve(s->ws, n.sum_out, ob, &dst, nullptr));
    HoloMatmulSeg sg = {dst, res, mm.n, 0};
    sg.all_reduce = 1;
    sg.b_constant = mm.b.slot < s->ws->slots.size() && s->ws->slots[mm.b.slot].constant;
    return holo_launch_matmul_multi(s->ctx, a, b, mm.m, mm.k, mm.n, mm.dtype, &sg, 1);
}

bool batchable_kind(uint16_t k) {
    return k == HOLO_K_KV_CACHE_WRITE || k == HOLO_K_ROTARY || k == HOLO_K_QUANTIZE_ROWS_I8 || k == HOLO_K_ADD || k == HOLO_K_MUL ||
           k == HOLO_K_ROPE_QUANTIZE_ROWS_I8;
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

}  // namespace

extern "C" int32_t holo_b200_label_bytes(const uint8_t* data, uint64_t len, uint8_t out71[71]) {
    if ((!data && len) || !out71) return holo_fail(HOLO_ERR_INIT, "null argument");
    holo_label_of_bytes(data, (size_t)len, out71);
    return HOLO_OK;
}

extern "C" int32_t holo_b200_label_derive(uint16_t opcode, const uint8_t* params, uint32_t params_len, const uint8_t* labels,
                                          uint32_t n_labels, uint8_t out71[71]) {
    if ((!params && params_len) || (!labels && n_labels) || !out71) return holo_fail(HOLO_ERR_INIT, "null argument");
    holo_label_derive(opcode, params, params_len, labels, n_labels, out71);
    return HOLO_OK;
}

extern "C" int32_t holo_b200_op_signature(const HoloKernelCall* call, uint16_t* opcode, uint8_t params64[64], uint32_t* params_len) {
    HoloOpSignature sig;
    if (!call || !holo_op_signature(*call, &sig))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: no operation signature for KernelCall variant %u", call ? call->kind : 0);
    if (opcode) *opcode = sig.opcode;
    if (params64) memcpy(params64, sig.params, sig.len);
    if (params_len) *params_len = sig.len;
    return HOLO_OK;
}

namespace {

int32_t run_calls(holo_b200_session* s) {
    for (const SessionNode& n : s->nodes) {
        if (n.matmul_reduce_add) HOLO_TRY(run_matmul_reduce_add(s, n));
        else if (n.reduce_add) HOLO_TRY(run_reduce_add(s, n));
        else if (n.merged >= 0) HOLO_TRY(run_merged(s, s->merged[n.merged]));
        else if (n.batch >= 0) HOLO_TRY(holo_launch_micro_batch(s->ctx, s->batches[n.batch].dev_ops, s->batches[n.batch].nops, s->batches[n.batch].total_ctas));
        else HOLO_TRY(holo_dispatch_internal(s->ctx, &n.call, s->ws));
    }
    return HOLO_OK;
}

}  // namespace

extern "C" int32_t holo_b200_session_load(holo_b200_ctx* ctx, const uint8_t* archive, uint64_t len, int32_t verify,
                                          holo_b200_session** out) {
    return holo_session_load_impl(ctx, archive, len, verify, nullptr, 0, out);
}

int32_t holo_session_load_impl(holo_b200_ctx* ctx, const uint8_t* archive, uint64_t len, int32_t verify, const HoloWeightProvider* provider,
                               uint64_t budget, holo_b200_session** out) {
    if (!ctx || !archive || !out) return holo_fail(HOLO_ERR_INIT, "backend init failed: null argument");
    HOLO_CUDA(cudaSetDevice(ctx->device));
    holo_b200_session* s = new holo_b200_session();
    s->ctx = ctx;
    s->addressed = (verify & HOLO_SESSION_ADDRESSED) != 0 || provider != nullptr;
    s->ad.residual_in_label = (verify & HOLO_SESSION_LABEL_RESIDUAL) != 0;
    if (provider) {
        s->ad.provider = *provider;
        s->ad.paged = true;
    }
    int32_t rc = holo_archive_parse(archive, len, (verify & HOLO_SESSION_VERIFY) != 0, &s->ar, provider != nullptr);
    if (rc != HOLO_OK) {
        delete s;
        return rc;
    }
    // execution order: ExecPlan levels, else one level in call order (session.rs:473)
    if (s->ar.exec_plan.empty()) {
        s->calls = s->ar.calls;
        s->call_level.assign(s->calls.size(), 0);
    } else {
        for (size_t li = 0; li < s->ar.exec_plan.size(); ++li)
            for (uint32_t idx : s->ar.exec_plan[li]) {
                s->calls.push_back(s->ar.calls[idx]);
                s->call_level.push_back((uint32_t)li);
            }
    }
    std::set<uint32_t> in_slots, out_slots;
    for (const HoloPort& p : s->ar.inputs) in_slots.insert(p.slot);
    for (const HoloPort& p : s->ar.outputs) out_slots.insert(p.slot);
    // a paged weight's length comes from the provider (session.rs:587-600)
    for (HoloConstant& k : s->ar.constants) {
        if (k.bytes || !k.by_reference) continue;
        const int64_t sz = provider && provider->size ? provider->size(provider->user, k.fingerprint) : -1;
        if (sz < 0) {
            delete s;
            return holo_fail(HOLO_ERR_INIT, "backend init failed: the weight provider does not have a weight the archive references");
        }
        k.len = (uint64_t)sz;
    }
    s->fused = fuse_matmul_epilogue(s->calls, s->call_level, out_slots);
    if (!s->addressed) s->rope_quant = fuse_rope_quantize(s->calls, s->call_level);
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
        for (uint32_t slot : const_slots)
            if (!written_slots.count(slot)) s->weight_slots.push_back(slot);
        if (s->addressed) {
            // one node per call: merged weights, batched launches and aliased slots all bake
            // device pointers in at load, which the label-keyed pool rebinds per walk
            for (const HoloKernelCall& c : s->calls) {
                SessionNode node;
                node.call = c;
                s->nodes.push_back(node);
            }
        } else {
            plan_sibling_merges(s, const_slots, written_slots);
            fuse_gated_pairs(s, out_slots);
            fuse_all_reduce_add(s, out_slots);
            fuse_matmul_reduce_add(s);
        }
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
        if (!s->addressed && in_slots.count(k.cache.slot) && out_slots.count(k.output.slot) && k.cache.offset == 0 &&
            k.output.offset == 0 && k.cache.slot != k.output.slot) {
            alias[k.output.slot] = k.cache.slot;
            need[k.cache.slot] = std::max(need[k.cache.slot], need[k.output.slot]);
            ++s->moved_in_place;
        }
    }
    // A paged session keeps load-time buffers only for what the pool cannot supply: resident constants
    // and the input ports (values written there by the caller); everything else lives in the pool.
    std::vector<uint8_t> lazy_slot(n_slots, 0), no_static(n_slots, 0);
    if (s->ad.paged) {
        std::fill(no_static.begin(), no_static.end(), 1);
        for (const HoloPort& p : s->ar.inputs) no_static[p.slot] = 0;
        for (const HoloConstant& k : s->ar.constants) {
            if (k.by_reference && !out_slots.count(k.slot)) lazy_slot[k.slot] = 1;
            else no_static[k.slot] = 0;
        }
    }
    rc = holo_b200_workspace_create(ctx, n_slots, &s->ws);
    for (uint32_t i = 0; rc == HOLO_OK && i < n_slots; ++i) {
        if (alias[i] >= 0 || no_static[i]) continue;
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
        if (lazy_slot[k.slot]) continue;   // paged in on first use
        const uint8_t* body = k.bytes;
        if (!body && provider && provider->get_range) body = (const uint8_t*)provider->get_range(provider->user, k.fingerprint, 0, k.len);
        if (!body && k.len) {
            rc = holo_fail(HOLO_ERR_INIT, "backend init failed: the weight provider could not serve a resident constant");
            break;
        }
        HoloBufferRef ref = {k.slot, 0, 0};
        rc = holo_b200_workspace_upload(s->ws, ref, body, k.len);
    }
    if (rc == HOLO_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = holo_fail(HOLO_ERR_INIT, "backend init failed: constant upload");
    if (rc == HOLO_OK) rc = build_merged_weights(s);
    if (rc == HOLO_OK && !s->addressed)
        for (uint32_t slot : s->weight_slots)
            if (slot < s->ws->slots.size() && s->ws->slots[slot].ptr) s->ws->slots[slot].constant = true;
    if (rc == HOLO_OK && !s->addressed) fuse_head_ops(s);
    if (rc == HOLO_OK && !s->addressed) rc = plan_micro_batches(s);
    if (rc == HOLO_OK && s->addressed) {
        s->ad.pool.reset();
        rc = holo_addressed_prepare(s, need);
        if (rc == HOLO_OK && s->ad.paged) s->ad.pool->set_lazy_budget(budget);
    }
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
    if (s->addressed) holo_addressed_destroy(s);   // hands the load-time buffers back to the workspace, frees the pool's own
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
    if (n_merged_calls) *n_merged_calls = s->merged_calls + s->batched_calls + s->head_fused + 2 * s->reduce_adds;
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
    if (s->addressed) {   // the plain walk of an addressed session runs on the load-time buffers
        if (s->ad.paged) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: a paged session executes through execute_addressed");
        holo_addressed_bind_static(s);
    }
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
