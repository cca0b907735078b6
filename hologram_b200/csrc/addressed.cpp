// Content-addressed execution over the device-resident label pool, paged weights, the memory-tier
// report and the pool's own C ABI. Host-side logic: every kernel it runs goes through the normal
// dispatch. Restates crates/hologram-exec/src/session.rs:942-1030 (execute_addressed, leases,
// intern / resolve), :1052-1289 (compute_and_label), :281-322 (compute_stealable), :1313-1370
// (kv_move_in_place), :243-270 + crates/hologram-exec/src/coherence.rs:78-225 (tiers).
#include <string.h>

#include <algorithm>
#include <map>

#include "blake3.h"
#include "session.h"

namespace {

std::string label_str(const uint8_t* l) { return std::string(reinterpret_cast<const char*>(l), HOLO_LABEL_BYTES); }

// ---- memory backends of the pool --------------------------------------------------------------
int dev_alloc(void* user, uint64_t bytes, void** out) {
    (void)user;
    return cudaMalloc(out, bytes) == cudaSuccess ? 0 : 1;
}
void dev_release(void* user, void* ptr) {
    (void)user;
    cudaFree(ptr);
}
int dev_zero(void* user, void* ptr, uint64_t bytes) {
    return cudaMemsetAsync(ptr, 0, bytes, static_cast<holo_b200_ctx*>(user)->stream) == cudaSuccess ? 0 : 1;
}
int dev_upload(void* user, void* dst, const void* host, uint64_t bytes) {
    return cudaMemcpyAsync(dst, host, bytes, cudaMemcpyHostToDevice, static_cast<holo_b200_ctx*>(user)->stream) == cudaSuccess ? 0 : 1;
}
int dev_download(void* user, void* host, const void* src, uint64_t bytes) {
    cudaStream_t st = static_cast<holo_b200_ctx*>(user)->stream;
    if (cudaMemcpyAsync(host, src, bytes, cudaMemcpyDeviceToHost, st) != cudaSuccess) return 1;
    return cudaStreamSynchronize(st) == cudaSuccess ? 0 : 1;
}
int dev_copy(void* user, void* dst, const void* src, uint64_t bytes) {
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<holo_b200_ctx*>(user)->stream) == cudaSuccess ? 0 : 1;
}
HoloPoolMemory device_memory(holo_b200_ctx* ctx) {
    HoloPoolMemory m;
    m.user = ctx;
    m.alloc = dev_alloc;
    m.release = dev_release;
    m.zero = dev_zero;
    m.upload = dev_upload;
    m.download = dev_download;
    m.copy = dev_copy;
    return m;
}

// plain host memory: the same table logic with no device (unit tests of the residency rules)
int host_alloc(void*, uint64_t bytes, void** out) {
    *out = malloc(bytes);
    return *out ? 0 : 1;
}
void host_release(void*, void* ptr) { free(ptr); }
int host_zero(void*, void* ptr, uint64_t bytes) {
    memset(ptr, 0, bytes);
    return 0;
}
int host_move(void*, void* dst, const void* src, uint64_t bytes) {
    memmove(dst, src, bytes);
    return 0;
}
HoloPoolMemory host_memory() {
    HoloPoolMemory m;
    m.alloc = host_alloc;
    m.release = host_release;
    m.zero = host_zero;
    m.upload = host_move;
    m.download = host_move;
    m.copy = host_move;
    return m;
}

const void* provider_range(void* user, const uint8_t fp[32], uint64_t offset, uint64_t size) {
    const HoloWeightProvider* p = static_cast<const HoloWeightProvider*>(user);
    return p && p->get_range ? p->get_range(p->user, fp, offset, size) : nullptr;
}

void sync_slot(holo_b200_session* s, uint32_t slot) {
    HoloSlot& sl = s->ws->slots[slot];
    sl.ptr = s->ad.pool->slot_ptr(slot);
    sl.bytes = s->ad.pool->slot_len(slot);
    sl.owned = false;   // the pool (or the load-time table) owns it
}

// Between walks an input port's slot is unbound: inputs enter an addressed session by label (intern_input), and a
// write through the workspace must never scribble over the pooled value that was bound there during the last walk.
void restore_input_ports(holo_b200_session* s) {
    for (const HoloPort& p : s->ar.inputs)
        if (p.slot < s->ws->slots.size()) s->ws->slots[p.slot] = HoloSlot();
}

// call_dtype (kernel_call.rs:1668-1760) for the served variants
uint8_t call_dtype(const HoloKernelCall& c) {
    const auto& u = c.u;
    if (holo_is_exact_unary(c.kind)) return u.unary.dtype;
    if (holo_is_exact_binary(c.kind)) return u.binary.dtype;
    switch (c.kind) {
        case HOLO_K_SIGMOID: case HOLO_K_TANH: case HOLO_K_GELU: case HOLO_K_SILU: case HOLO_K_EXP: case HOLO_K_ERF: return u.unary.dtype;
        case HOLO_K_ADD: case HOLO_K_MUL: case HOLO_K_CONCAT: return u.binary.dtype;
        case HOLO_K_MATMUL: case HOLO_K_MATMUL_ACTIVATION: case HOLO_K_MATMUL_ADD: case HOLO_K_MATMUL_ADD_ACTIVATION: return u.matmul.dtype;
        case HOLO_K_MATMUL_DEQUANT_PLAIN: case HOLO_K_MATMUL_DEQUANT: case HOLO_K_MATMUL_DEQUANT_CODEBOOK: return u.matmul_dequant.dtype;
        case HOLO_K_LAYER_NORM: case HOLO_K_RMS_NORM: case HOLO_K_ADD_RMS_NORM: return u.norm.dtype;
        case HOLO_K_REDUCE_SUM: case HOLO_K_REDUCE_MEAN: case HOLO_K_REDUCE_PROD: case HOLO_K_REDUCE_MIN: case HOLO_K_REDUCE_MAX: return u.reduce.dtype;
        case HOLO_K_RESHAPE: case HOLO_K_SLICE: return u.layout.dtype;
        case HOLO_K_TRANSPOSE: return u.transpose.dtype;
        case HOLO_K_SOFTMAX: return u.softmax.dtype;
        case HOLO_K_ATTENTION: return u.attention.dtype;
        case HOLO_K_EXPAND: return u.expand.dtype;
        case HOLO_K_ROTARY: return u.rope.dtype;
        case HOLO_K_WHERE: return u.where.dtype;
        case HOLO_K_DEQUANTIZE: return u.dequantize.dtype;
        case HOLO_K_BROADCAST_BINARY: return u.broadcast_binary.dtype;
        case HOLO_K_DEQUANT_ACTIVATION: return u.dequant_activation.dtype;
        case HOLO_K_GATHER: return u.gather.dtype;
        case HOLO_K_CAST: return u.cast.dst_dtype;
        case HOLO_K_DECODE_ATTENTION: return u.decode_attention.dtype;
        case HOLO_K_KV_CACHE_WRITE: return HOLO_DTYPE_U8;
        case HOLO_K_DECODE_ATTENTION_VALID: return u.decode_attention_valid.dtype;
        case HOLO_K_QUANTIZE_ROWS_I8: return u.quantize_rows_i8.dtype;
        case HOLO_K_DECODE_ATTENTION_VALID_Q8: return u.decode_attention_valid_q8.dtype;
        case HOLO_K_ALL_REDUCE: return u.all_reduce.dtype;
        case HOLO_K_ROPE_QUANTIZE_ROWS_I8: return u.rope_quantize.dtype;
        default: return HOLO_DTYPE_F32;
    }
}

// is_layout_only_call (session.rs:255-270)
bool layout_only(uint16_t k) {
    return k == HOLO_K_RESHAPE || k == HOLO_K_TRANSPOSE || k == HOLO_K_CONCAT || k == HOLO_K_SLICE || k == HOLO_K_EXPAND || k == HOLO_K_GATHER ||
           k == HOLO_K_KV_CACHE_WRITE;
}

enum { TIER_CPU_L1 = 0, TIER_CPU_L2 = 1, TIER_CPU_MAIN = 2, TIER_DEVICE = 3 };

// MemoryTier::from_witt (memory_tier.rs:41-51) over the dtype's bit width (call_tier, session.rs:243-250)
int call_tier(const HoloKernelCall& c) {
    if (layout_only(c.kind)) return TIER_CPU_MAIN;
    size_t bpe = holo_dtype_size(call_dtype(c));
    if (bpe == 0) bpe = 1;
    const size_t bits = bpe * 8;
    return bits <= 8 ? TIER_CPU_L1 : bits <= 16 ? TIER_CPU_L2 : bits <= 24 ? TIER_CPU_MAIN : TIER_DEVICE;
}

}  // namespace

// ---- session set-up -----------------------------------------------------------------------------
int32_t holo_addressed_prepare(holo_b200_session* s, const std::vector<uint64_t>& need) {
    HoloAddressed& ad = s->ad;
    const size_t n_slots = s->ws->slots.size();
    ad.slot_need.assign(need.begin(), need.end());
    ad.static_binding = s->ws->slots;
    ad.slot_label_init.assign(n_slots, std::string());
    ad.is_output_slot.assign(n_slots, 0);
    ad.is_input_slot.assign(n_slots, 0);
    for (const HoloPort& p : s->ar.outputs) ad.is_output_slot[p.slot] = 1;
    for (const HoloPort& p : s->ar.inputs) ad.is_input_slot[p.slot] = 1;
    ad.pool.reset(new HoloPool(device_memory(s->ctx)));
    // constants are leaves: their label is the label of their bytes; for a weight stored by reference
    // that is its fingerprint rendered as a label (address.rs:63-74), no body needed
    for (const HoloConstant& k : s->ar.constants) {
        uint8_t l[HOLO_LABEL_BYTES];
        if (k.by_reference) holo_label_from_digest(k.fingerprint, l);
        else holo_label_of_bytes(k.bytes, k.len, l);
        const std::string label = label_str(l);
        const bool lazy = ad.paged && k.by_reference && !ad.is_output_slot[k.slot];
        if (lazy) {
            ad.pool->pin_lazy(label, k.fingerprint, k.len);
            ad.lazy_slots[k.slot] = label;
        } else {
            ad.pool->pin_external(label, ad.static_binding[k.slot].ptr, k.len);
        }
        ad.slot_label_init[k.slot] = label;
        ad.const_bindings.push_back({k.slot, label});
    }
    ad.meta.resize(s->calls.size());
    for (size_t i = 0; i < s->calls.size(); ++i) {
        HoloAddressed::NodeMeta& m = ad.meta[i];
        const HoloKernelCall& c = s->calls[i];
        uint32_t out = HOLO_NO_SLOT;
        m.addressable = holo_op_signature(c, &m.sig) && holo_call_operands(c, &m.inputs, &out, ad.residual_in_label);
        if (m.addressable) {
            m.outputs.push_back(out);
        } else if (c.kind == HOLO_K_QUANTIZE_ROWS_I8) {
            // two outputs: codes take the plain derivation, scales the derivation with an index byte
            m.addressable = holo_op_signature(c, &m.sig);
            m.inputs = {c.u.quantize_rows_i8.input.slot};
            m.outputs = {c.u.quantize_rows_i8.codes.slot, c.u.quantize_rows_i8.scales.slot};
        } else {
            HoloKernelCall tmp = c;
            HoloRefList refs;
            if (holo_collect_refs(&tmp, &refs))
                for (int r = 0; r < refs.n; ++r) {
                    if (refs.refs[r]->slot == HOLO_NO_SLOT) continue;
                    if (refs.written[r]) m.outputs.push_back(refs.refs[r]->slot);
                    else m.inputs.push_back(refs.refs[r]->slot);
                }
            // an all-reduce rewrites its buffer where it lies: the slot keeps its binding, the value loses its label
            m.in_place = c.kind == HOLO_K_ALL_REDUCE;
        }
    }
    // compute_stealable (session.rs:281-322): a KvCacheWrite may mutate the resident cache buffer only if
    // every other call that touches the cache slot (as operand or as output) runs strictly before it
    ad.stealable.assign(s->calls.size(), 0);
    for (size_t i = 0; i < s->calls.size(); ++i) {
        if (s->calls[i].kind != HOLO_K_KV_CACHE_WRITE) continue;
        const uint32_t cache_slot = s->calls[i].u.kv_cache_write.cache.slot;
        bool ok = true;
        for (size_t j = 0; j < s->calls.size() && ok; ++j) {
            if (j == i) continue;
            const HoloAddressed::NodeMeta& m = ad.meta[j];
            const bool touches = std::find(m.inputs.begin(), m.inputs.end(), cache_slot) != m.inputs.end() ||
                                 std::find(m.outputs.begin(), m.outputs.end(), cache_slot) != m.outputs.end();
            if (touches && !(j < i)) ok = false;
        }
        ad.stealable[i] = ok ? 1 : 0;
    }
    return HOLO_OK;
}

void holo_addressed_bind_static(holo_b200_session* s) {
    for (size_t i = 0; i < s->ad.static_binding.size() && i < s->ws->slots.size(); ++i) {
        s->ws->slots[i].ptr = s->ad.static_binding[i].ptr;
        s->ws->slots[i].bytes = s->ad.static_binding[i].bytes;
        s->ws->slots[i].owned = false;
    }
}

void holo_addressed_destroy(holo_b200_session* s) {
    // hand the load-time buffers back to the workspace before it frees them, then the pool's own
    for (size_t i = 0; i < s->ad.static_binding.size() && i < s->ws->slots.size(); ++i) s->ws->slots[i] = s->ad.static_binding[i];
    s->ad.pool.reset();
}

// ---- the walk -----------------------------------------------------------------------------------
extern "C" int32_t holo_b200_session_execute_addressed(holo_b200_session* s, const uint8_t* input_labels, uint32_t n_inputs,
                                                       uint8_t* output_labels, uint32_t n_outputs, HoloAddressedStats* stats) {
    if (!s) return holo_fail(HOLO_ERR_INIT, "null session");
    if (!s->addressed) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: the session was not loaded with HOLO_SESSION_ADDRESSED");
    if (n_inputs != s->ar.inputs.size() || n_outputs != s->ar.outputs.size() || (!input_labels && n_inputs) || (!output_labels && n_outputs))
        return holo_fail(HOLO_ERR_SHAPE_MISMATCH, "shape mismatch: execute_addressed takes %zu input labels and %zu output labels",
                         s->ar.inputs.size(), s->ar.outputs.size());
    HOLO_CUDA(cudaSetDevice(s->ctx->device));
    HoloAddressed& ad = s->ad;
    HoloPool& pool = *ad.pool;
    HoloAddressedStats st = {};
    const size_t n_slots = s->ws->slots.size();

    // whole-graph memo (session.rs:63-111): the same input labels give the same output labels; a hit
    // counts only while every output is still resident. The outputs are bound to their slots so that
    // they can be read through the workspace as after a walk.
    const std::string key(reinterpret_cast<const char*>(input_labels), (size_t)n_inputs * HOLO_LABEL_BYTES);
    auto hit = ad.memo.find(key);
    if (hit != ad.memo.end()) {
        bool resident = true;
        for (uint32_t o = 0; o < n_outputs && resident; ++o)
            resident = pool.resident(hit->second.first.substr((size_t)o * HOLO_LABEL_BYTES, HOLO_LABEL_BYTES));
        if (resident) {
            hit->second.second = ++ad.memo_tick;
            for (uint32_t o = 0; o < n_outputs; ++o) {
                const uint32_t slot = s->ar.outputs[o].slot;
                pool.bind_resident(slot, hit->second.first.substr((size_t)o * HOLO_LABEL_BYTES, HOLO_LABEL_BYTES));
                sync_slot(s, slot);
            }
            memcpy(output_labels, hit->second.first.data(), (size_t)n_outputs * HOLO_LABEL_BYTES);
            restore_input_ports(s);
            ad.last_dispatched = 0;
            ad.last_skipped = (uint32_t)s->calls.size();
            ad.last_moved = 0;
            st.memo_hit = 1;
            st.skipped = ad.last_skipped;
            st.pool_bytes = pool.owned_bytes();
            st.paged_in = (uint32_t)pool.pages_in();
            if (stats) *stats = st;
            return HOLO_OK;
        }
    }

    // Refuse before any state change (session.rs:959-971): the rotation below ages the pool, so a call that
    // cannot bind must not rotate. Bindability is checked against what survives the rotation: pinned, the
    // current generation, leases, paged-in weights. A label living only in the previous generation is one
    // rotation from reclamation: intern the value again (that promotes it) or feed a fresh output label.
    std::vector<std::string> in_label(n_inputs);
    for (uint32_t i = 0; i < n_inputs; ++i) {
        in_label[i] = label_str(input_labels + (size_t)i * HOLO_LABEL_BYTES);
        if (!pool.bindable_input(in_label[i]))
            return holo_fail(HOLO_ERR_SHAPE_MISMATCH, "shape mismatch: input %u (%s) is not resident under its label: intern it, or pass a label a walk returned",
                             i, s->ar.inputs[i].name.c_str());
    }

    pool.rebind_reset(n_slots);
    for (size_t i = 0; i < n_slots; ++i) s->ws->slots[i] = HoloSlot();
    for (auto& cb : ad.const_bindings) {
        if (ad.lazy_slots.count(cb.first)) continue;   // paged in right before the call that reads it
        pool.bind_resident(cb.first, cb.second);
        sync_slot(s, cb.first);
    }
    std::vector<std::string> label = ad.slot_label_init;
    for (uint32_t i = 0; i < n_inputs; ++i) {
        const uint32_t slot = s->ar.inputs[i].slot;
        if (!pool.bind_resident(slot, in_label[i])) {
            return holo_fail(HOLO_ERR_SHAPE_MISMATCH, "shape mismatch: input %u could not be bound by its label", i);
        }
        sync_slot(s, slot);
        label[slot] = in_label[i];
    }

    std::vector<std::string> out_witnessed(n_slots);
    for (size_t ci = 0; ci < s->calls.size(); ++ci) {
        const HoloAddressed::NodeMeta& m = ad.meta[ci];
        const HoloKernelCall& call = s->calls[ci];
        // operand labels, in kernel order; a commutative op sorts them (session.rs:1095-1102)
        std::vector<std::string> in;
        bool addressable = m.addressable;
        for (uint32_t sl : m.inputs) {
            if (!addressable) break;
            if (label[sl].empty()) { addressable = false; break; }
            in.push_back(label[sl]);
        }
        const std::string cache_label = (addressable && !in.empty()) ? in[0] : std::string();
        if (addressable && m.sig.commutative) std::sort(in.begin(), in.end());
        std::string cat;
        for (const std::string& l : in) cat += l;
        auto derive = [&](size_t o, bool boundary) {
            uint8_t params[80], l[HOLO_LABEL_BYTES];
            memcpy(params, m.sig.params, m.sig.len);
            size_t plen = m.sig.len;
            if (o > 0) params[plen++] = (uint8_t)o;   // a second result of one call: the same derivation with an index byte
            if (boundary) holo_label_derive_boundary(m.sig.opcode, params, plen, reinterpret_cast<const uint8_t*>(cat.data()), in.size(), l);
            else holo_label_derive(m.sig.opcode, params, plen, reinterpret_cast<const uint8_t*>(cat.data()), in.size(), l);
            return label_str(l);
        };
        std::vector<std::string> out_label(m.outputs.size());
        if (addressable)
            for (size_t o = 0; o < m.outputs.size(); ++o)
                // a reshape relabels nothing: its value is its input's (session.rs:1107-1114)
                out_label[o] = (call.kind == HOLO_K_RESHAPE && !in.empty()) ? in[0] : derive(o, false);

        // interior reuse: every result resident and none a graph output -> bind, do not dispatch
        bool reuse = addressable && !m.outputs.empty();
        for (size_t o = 0; o < m.outputs.size() && reuse; ++o) reuse = !ad.is_output_slot[m.outputs[o]] && pool.resident(out_label[o]);
        if (reuse) {
            for (size_t o = 0; o < m.outputs.size(); ++o) {
                pool.bind_resident(m.outputs[o], out_label[o]);
                sync_slot(s, m.outputs[o]);
                label[m.outputs[o]] = out_label[o];
            }
            ++st.skipped;
            continue;
        }

        // KvCacheWrite in-place move (session.rs:1163-1194, 1313-1370): when the plan admits it and the
        // cache value is an unaliased transient resident, its own buffer becomes the output (the cache
        // label is retired) and only the new rows are written
        bool moved = false;
        if (ad.stealable[ci] && addressable && call.kind == HOLO_K_KV_CACHE_WRITE && m.outputs.size() == 1) {
            const HoloKvCacheWriteCall& kc = call.u.kv_cache_write;
            const uint32_t out_slot = m.outputs[0];
            const uint64_t need_bytes = (uint64_t)kc.planes * kc.bucket_rows * kc.row_bytes;
            const size_t cbi = pool.find(cache_label);
            if (kc.bucket_rows != 0 && kc.row_bytes != 0 && kc.new_rows <= kc.bucket_rows && cbi != HoloPool::UNBOUND &&
                pool.buffer_len(cbi) >= need_bytes && kc.cache.offset == 0 && kc.output.offset == 0) {
                std::vector<size_t> allowed(m.inputs.begin(), m.inputs.end());
                allowed.push_back(out_slot);
                const size_t bi = pool.steal_transient(cache_label, allowed);
                if (bi != HoloPool::UNBOUND) {
                    pool.bind_buffer(out_slot, bi);   // the cache slot stays bound to the same buffer: the kernel takes its in-place form
                    sync_slot(s, out_slot);
                    moved = true;
                }
            }
        }
        if (!moved) {
            // paged session: page in and bind this call's lazy operands as one group, right before the
            // kernel reads them (session.rs:1196-1224)
            if (ad.paged && !ad.lazy_slots.empty()) {
                std::vector<std::pair<size_t, std::string>> group;
                for (uint32_t sl : m.inputs) {
                    auto lz = ad.lazy_slots.find(sl);
                    if (lz != ad.lazy_slots.end()) group.push_back({sl, lz->second});
                }
                if (!group.empty()) {
                    if (!pool.page_and_bind_group(group, provider_range, &ad.provider))
                        return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: a paged weight could not be brought in (provider or memory)");
                    for (auto& g : group) sync_slot(s, (uint32_t)g.first);
                }
            }
            for (size_t o = 0; o < m.outputs.size(); ++o) {
                const uint32_t slot = m.outputs[o];
                if (m.in_place) {
                    // the value is rewritten where it lies: the buffer must stop answering to its old label,
                    // or be left alone (copied) when something else still owns it
                    const size_t bi = pool.bound(slot);
                    if (bi == HoloPool::UNBOUND) return holo_fail_slot(slot, "slot is not bound");
                    if (!pool.disown_transient(bi)) {
                        const void* src = pool.buffer_ptr(bi);
                        const uint64_t nb = pool.buffer_len(bi);
                        const size_t fresh = pool.bind_fresh(slot, nb);
                        if (fresh == HoloPool::UNBOUND) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: the label pool could not allocate %llu bytes", (unsigned long long)nb);
                        if (nb) HOLO_CUDA(cudaMemcpyAsync(pool.buffer_ptr(fresh), src, nb, cudaMemcpyDeviceToDevice, s->ctx->stream));
                    }
                } else {
                    const uint64_t nb = slot < ad.slot_need.size() ? ad.slot_need[slot] : 64;
                    if (pool.bind_fresh(slot, nb) == HoloPool::UNBOUND)
                        return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: the label pool could not allocate %llu bytes", (unsigned long long)nb);
                }
                sync_slot(s, slot);
            }
        }
        HOLO_TRY(holo_dispatch_internal(s->ctx, &call, s->ws));
        if (moved) {
            ++st.moved;
            ++st.skipped;
        } else {
            ++st.dispatched;
        }
        for (size_t o = 0; o < m.outputs.size(); ++o) {
            const uint32_t slot = m.outputs[o];
            out_witnessed[slot].clear();   // whatever an earlier producer of this slot was retained under no longer names it
            if (!addressable) {
                label[slot].clear();
                continue;
            }
            if (ad.is_output_slot[slot]) {
                // a graph output is retained under the boundary form; the slot keeps the cheap label for
                // downstream derivations (session.rs:1234-1252)
                const std::string w = derive(o, true);
                pool.retain(slot, w);
                out_witnessed[slot] = w;
            } else {
                pool.retain(slot, out_label[o]);
            }
            label[slot] = out_label[o];
        }
    }

    // output labels; an output whose value has no derivable label is addressed by its logical bytes,
    // the only place a result is read back and hashed (session.rs:1262-1280)
    std::string outs;
    for (uint32_t o = 0; o < n_outputs; ++o) {
        const HoloPort& port = s->ar.outputs[o];
        std::string l = out_witnessed[port.slot];
        if (l.empty()) {
            const size_t bi = pool.bound(port.slot);
            if (bi == HoloPool::UNBOUND) return holo_fail_slot(port.slot, "output slot is not bound after the walk");
            const uint64_t nb = std::min<uint64_t>(port.element_count * holo_dtype_size(port.dtype), pool.buffer_len(bi));
            std::vector<uint8_t> host(nb);
            HOLO_CUDA(cudaMemcpyAsync(host.data(), pool.buffer_ptr(bi), nb, cudaMemcpyDeviceToHost, s->ctx->stream));
            HOLO_CUDA(cudaStreamSynchronize(s->ctx->stream));
            uint8_t lb[HOLO_LABEL_BYTES];
            holo_label_of_bytes(host.data(), nb, lb);
            l = label_str(lb);
            pool.retain(port.slot, l);
        }
        memcpy(output_labels + (size_t)o * HOLO_LABEL_BYTES, l.data(), HOLO_LABEL_BYTES);
        outs += l;
    }
    if (ad.memo.size() >= 1024 && !ad.memo.count(key)) {   // least recently used entry goes (session.rs:93-105)
        auto lru = ad.memo.begin();
        for (auto it = ad.memo.begin(); it != ad.memo.end(); ++it)
            if (it->second.second < lru->second.second) lru = it;
        ad.memo.erase(lru);
    }
    ad.memo[key] = {outs, ++ad.memo_tick};
    restore_input_ports(s);
    ad.last_dispatched = st.dispatched;
    ad.last_skipped = st.skipped;
    ad.last_moved = st.moved;
    st.pool_bytes = pool.owned_bytes();
    st.paged_in = (uint32_t)pool.pages_in();
    if (stats) *stats = st;
    return HOLO_OK;
}

extern "C" int32_t holo_b200_session_intern_input(holo_b200_session* s, const void* host, uint64_t len, uint8_t out71[71]) {
    if (!s || (!host && len) || !out71) return holo_fail(HOLO_ERR_INIT, "null argument");
    if (!s->addressed) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: the session was not loaded with HOLO_SESSION_ADDRESSED");
    HOLO_CUDA(cudaSetDevice(s->ctx->device));
    holo_label_of_bytes(static_cast<const uint8_t*>(host), (size_t)len, out71);
    if (!s->ad.pool->store_unbound(label_str(out71), host, len))
        return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: the label pool could not store %llu bytes", (unsigned long long)len);
    // the copy reads pageable or pinned host memory asynchronously: the caller may reuse `host` when this returns
    HOLO_CUDA(cudaStreamSynchronize(s->ctx->stream));
    return HOLO_OK;
}

extern "C" int32_t holo_b200_session_resolve(holo_b200_session* s, const uint8_t label71[71], void* host, uint64_t cap, uint64_t* len,
                                             int32_t* resident) {
    if (!s || !label71) return holo_fail(HOLO_ERR_INIT, "null argument");
    if (!s->addressed) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: the session was not loaded with HOLO_SESSION_ADDRESSED");
    HOLO_CUDA(cudaSetDevice(s->ctx->device));
    const std::string label = label_str(label71);
    const bool here = s->ad.pool->find(label) != HoloPool::UNBOUND;
    if (resident) *resident = here ? 1 : 0;
    if (!here) {
        if (len) *len = 0;
        return HOLO_OK;
    }
    if (!s->ad.pool->resolve(label, host, host ? cap : 0, len)) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: reading a pooled value back");
    return HOLO_OK;
}

extern "C" int32_t holo_b200_session_retain_label(holo_b200_session* s, const uint8_t label71[71], int32_t* ok) {
    if (!s || !label71) return holo_fail(HOLO_ERR_INIT, "null argument");
    if (!s->addressed) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: the session was not loaded with HOLO_SESSION_ADDRESSED");
    const bool r = s->ad.pool->lease(label_str(label71));
    if (ok) *ok = r ? 1 : 0;
    return HOLO_OK;
}

extern "C" int32_t holo_b200_session_release_label(holo_b200_session* s, const uint8_t label71[71], int32_t* ok) {
    if (!s || !label71) return holo_fail(HOLO_ERR_INIT, "null argument");
    if (!s->addressed) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: the session was not loaded with HOLO_SESSION_ADDRESSED");
    const bool r = s->ad.pool->release(label_str(label71));
    if (ok) *ok = r ? 1 : 0;
    return HOLO_OK;
}

extern "C" uint32_t holo_b200_session_leased_count(holo_b200_session* s) {
    return s && s->addressed ? (uint32_t)s->ad.pool->leased_len() : 0;
}

extern "C" int32_t holo_b200_label_derive_boundary(uint16_t opcode, const uint8_t* params, uint32_t params_len, const uint8_t* labels,
                                                   uint32_t n_labels, uint8_t out71[71]) {
    if ((!params && params_len) || (!labels && n_labels) || !out71) return holo_fail(HOLO_ERR_INIT, "null argument");
    if (!holo_label_derive_boundary(opcode, params, params_len, labels, n_labels, out71))
        return holo_fail(HOLO_ERR_SHAPE_MISMATCH, "shape mismatch: an operand is not a well-formed blake3 label");
    return HOLO_OK;
}

extern "C" int32_t holo_b200_session_load_paged(holo_b200_ctx* ctx, const uint8_t* archive, uint64_t len, int32_t verify,
                                                const HoloWeightProvider* provider, uint64_t budget_bytes, holo_b200_session** out) {
    if (!provider || !provider->size || !provider->get_range) return holo_fail(HOLO_ERR_INIT, "backend init failed: load_paged needs a weight provider");
    return holo_session_load_impl(ctx, archive, len, verify | HOLO_SESSION_ADDRESSED, provider, budget_bytes, out);
}

// ---- memory tiers ---------------------------------------------------------------------------------
extern "C" int32_t holo_b200_session_tier_report(holo_b200_session* s, int32_t policy, HoloTierReport* out) {
    if (!s || !out) return holo_fail(HOLO_ERR_INIT, "null argument");
    if (policy < HOLO_TIER_COMPILED || policy > HOLO_TIER_FORCE_ALL_DEVICE) return holo_fail(HOLO_ERR_SHAPE_MISMATCH, "shape mismatch: unknown tier policy %d", policy);
    memset(out, 0, sizeof *out);
    const size_t n = s->calls.size();
    std::vector<int> tier(n);
    for (size_t i = 0; i < n; ++i) {
        const int t = call_tier(s->calls[i]);
        tier[i] = policy == HOLO_TIER_FORCE_ALL_CPU ? TIER_CPU_MAIN : policy == HOLO_TIER_FORCE_ALL_DEVICE ? TIER_DEVICE : t;   // TierPolicy::apply (coherence.rs:141-151)
        switch (tier[i]) {
            case TIER_CPU_L1: ++out->cpu_l1_calls; break;
            case TIER_CPU_L2: ++out->cpu_l2_calls; break;
            case TIER_CPU_MAIN: ++out->cpu_main_calls; break;
            default: ++out->device_calls; break;
        }
    }
    // build_migration_schedule (coherence.rs:168-225): every slot starts on the CPU; before a level, a slot a
    // device call reads that the CPU owns moves up (and becomes shared), a slot a CPU call reads that the device
    // owns moves down; after the level every written slot belongs to its writer's side
    uint32_t n_slots = (uint32_t)s->ws->slots.size();
    std::vector<uint8_t> owner(n_slots, 0);   // 0 cpu, 1 device, 2 shared
    std::map<uint32_t, std::vector<size_t>> levels;
    for (size_t i = 0; i < n; ++i) levels[i < s->call_level.size() ? s->call_level[i] : 0].push_back(i);
    for (auto& lv : levels) {
        uint32_t moved = 0;
        std::vector<std::vector<uint32_t>> ins(lv.second.size()), outs(lv.second.size());
        for (size_t q = 0; q < lv.second.size(); ++q) {
            HoloKernelCall tmp = s->calls[lv.second[q]];
            HoloRefList refs;
            if (!holo_collect_refs(&tmp, &refs)) continue;
            for (int r = 0; r < refs.n; ++r) {
                const uint32_t slot = refs.refs[r]->slot;
                if (slot == HOLO_NO_SLOT || slot >= n_slots) continue;
                (refs.written[r] ? outs[q] : ins[q]).push_back(slot);
            }
        }
        for (size_t q = 0; q < lv.second.size(); ++q) {
            const bool needs_device = tier[lv.second[q]] == TIER_DEVICE;
            for (uint32_t slot : ins[q]) {
                if (needs_device && owner[slot] == 0) { ++moved; owner[slot] = 2; }
                else if (!needs_device && owner[slot] == 1) { ++moved; owner[slot] = 2; }
            }
        }
        for (size_t q = 0; q < lv.second.size(); ++q)
            for (uint32_t slot : outs[q]) owner[slot] = tier[lv.second[q]] == TIER_DEVICE ? 1 : 0;
        out->total_migration_slots += moved;
        if (moved) ++out->levels_with_migrations;
    }
    return HOLO_OK;
}

// ---- the pool's own C ABI -------------------------------------------------------------------------
struct holo_b200_pool {
    holo_b200_ctx* ctx = nullptr;
    std::unique_ptr<HoloPool> pool;
};

extern "C" int32_t holo_b200_pool_create(holo_b200_ctx* ctx, holo_b200_pool** out) {
    if (!out) return holo_fail(HOLO_ERR_INIT, "null argument");
    if (ctx) HOLO_CUDA(cudaSetDevice(ctx->device));
    holo_b200_pool* p = new holo_b200_pool();
    p->ctx = ctx;
    p->pool.reset(new HoloPool(ctx ? device_memory(ctx) : host_memory()));
    *out = p;
    return HOLO_OK;
}

extern "C" void holo_b200_pool_destroy(holo_b200_pool* p) {
    if (!p) return;
    if (p->ctx) {
        cudaSetDevice(p->ctx->device);
        cudaStreamSynchronize(p->ctx->stream);
    }
    delete p;
}

#define POOL_ARG(p)                                                  \
    if (!(p)) return holo_fail(HOLO_ERR_INIT, "null pool");          \
    if ((p)->ctx) HOLO_CUDA(cudaSetDevice((p)->ctx->device));

extern "C" int32_t holo_b200_pool_rebind_reset(holo_b200_pool* p, uint32_t n_slots) {
    POOL_ARG(p);
    p->pool->rebind_reset(n_slots);
    return HOLO_OK;
}
extern "C" int32_t holo_b200_pool_store_unbound(holo_b200_pool* p, const uint8_t label71[71], const void* host, uint64_t len) {
    POOL_ARG(p);
    if (!p->pool->store_unbound(label_str(label71), host, len)) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: the pool could not store the value");
    if (p->ctx) HOLO_CUDA(cudaStreamSynchronize(p->ctx->stream));
    return HOLO_OK;
}
extern "C" int32_t holo_b200_pool_pin_bytes(holo_b200_pool* p, const uint8_t label71[71], const void* host, uint64_t len) {
    POOL_ARG(p);
    if (!p->pool->pin_bytes(label_str(label71), host, len)) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: the pool could not pin the value");
    if (p->ctx) HOLO_CUDA(cudaStreamSynchronize(p->ctx->stream));
    return HOLO_OK;
}
extern "C" int32_t holo_b200_pool_bind_fresh(holo_b200_pool* p, uint32_t slot, uint64_t len) {
    POOL_ARG(p);
    if (p->pool->bind_fresh(slot, len) == HoloPool::UNBOUND) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: the pool could not allocate");
    return HOLO_OK;
}
extern "C" int32_t holo_b200_pool_bind_resident(holo_b200_pool* p, uint32_t slot, const uint8_t label71[71]) {
    POOL_ARG(p);
    return p->pool->bind_resident(slot, label_str(label71)) ? 1 : 0;
}
extern "C" int32_t holo_b200_pool_retain(holo_b200_pool* p, uint32_t slot, const uint8_t label71[71]) {
    POOL_ARG(p);
    p->pool->retain(slot, label_str(label71));
    return HOLO_OK;
}
extern "C" int32_t holo_b200_pool_steal_transient(holo_b200_pool* p, const uint8_t label71[71], const uint32_t* allowed_slots, uint32_t n_allowed,
                                                  uint32_t out_slot) {
    POOL_ARG(p);
    std::vector<size_t> allowed(allowed_slots, allowed_slots + n_allowed);
    const size_t bi = p->pool->steal_transient(label_str(label71), allowed);
    if (bi == HoloPool::UNBOUND) return 0;
    p->pool->bind_buffer(out_slot, bi);
    return 1;
}
extern "C" int32_t holo_b200_pool_lease(holo_b200_pool* p, const uint8_t label71[71]) {
    POOL_ARG(p);
    return p->pool->lease(label_str(label71)) ? 1 : 0;
}
extern "C" int32_t holo_b200_pool_release(holo_b200_pool* p, const uint8_t label71[71]) {
    POOL_ARG(p);
    return p->pool->release(label_str(label71)) ? 1 : 0;
}
extern "C" int32_t holo_b200_pool_resident(holo_b200_pool* p, const uint8_t label71[71]) {
    POOL_ARG(p);
    return p->pool->resident(label_str(label71)) ? 1 : 0;
}
extern "C" int32_t holo_b200_pool_bindable_input(holo_b200_pool* p, const uint8_t label71[71]) {
    POOL_ARG(p);
    return p->pool->bindable_input(label_str(label71)) ? 1 : 0;
}
extern "C" int32_t holo_b200_pool_resolve(holo_b200_pool* p, const uint8_t label71[71], void* host, uint64_t cap, uint64_t* len) {
    POOL_ARG(p);
    return p->pool->resolve(label_str(label71), host, host ? cap : 0, len) ? 1 : 0;
}
extern "C" int32_t holo_b200_pool_slot(holo_b200_pool* p, uint32_t slot, void** ptr, uint64_t* len) {
    POOL_ARG(p);
    if (p->pool->bound(slot) == HoloPool::UNBOUND) return 0;
    if (ptr) *ptr = p->pool->slot_ptr(slot);
    if (len) *len = p->pool->slot_len(slot);
    return 1;
}
extern "C" int32_t holo_b200_pool_write_slot(holo_b200_pool* p, uint32_t slot, const void* host, uint64_t len) {
    POOL_ARG(p);
    if (p->pool->bound(slot) == HoloPool::UNBOUND || len > p->pool->slot_len(slot)) return holo_fail_slot(slot, "slot is unbound or shorter than the write");
    if (p->ctx) {
        HOLO_CUDA(cudaMemcpyAsync(p->pool->slot_ptr(slot), host, len, cudaMemcpyHostToDevice, p->ctx->stream));
        HOLO_CUDA(cudaStreamSynchronize(p->ctx->stream));
    } else {
        memcpy(p->pool->slot_ptr(slot), host, len);
    }
    return HOLO_OK;
}
extern "C" int32_t holo_b200_pool_set_lazy_budget(holo_b200_pool* p, uint64_t bytes) {
    POOL_ARG(p);
    p->pool->set_lazy_budget(bytes);
    return HOLO_OK;
}
extern "C" int32_t holo_b200_pool_pin_lazy(holo_b200_pool* p, const uint8_t label71[71], const uint8_t fingerprint[32], uint64_t size) {
    POOL_ARG(p);
    p->pool->pin_lazy(label_str(label71), fingerprint, size);
    return HOLO_OK;
}
extern "C" int32_t holo_b200_pool_page_and_bind(holo_b200_pool* p, const uint32_t* slots, const uint8_t* labels, uint32_t n,
                                                const HoloWeightProvider* provider) {
    POOL_ARG(p);
    std::vector<std::pair<size_t, std::string>> group;
    for (uint32_t i = 0; i < n; ++i) group.push_back({slots[i], label_str(labels + (size_t)i * HOLO_LABEL_BYTES)});
    const bool ok = p->pool->page_and_bind_group(group, provider_range, const_cast<HoloWeightProvider*>(provider));
    if (p->ctx) HOLO_CUDA(cudaStreamSynchronize(p->ctx->stream));
    return ok ? 1 : 0;
}
extern "C" int32_t holo_b200_pool_stats(holo_b200_pool* p, HoloPoolStats* out) {
    POOL_ARG(p);
    if (!out) return holo_fail(HOLO_ERR_INIT, "null argument");
    out->owned_bytes = p->pool->owned_bytes();
    out->lazy_resident_bytes = p->pool->lazy_resident_bytes();
    out->pages_in = p->pool->pages_in();
    out->leased = (uint32_t)p->pool->leased_len();
    out->transient = (uint32_t)p->pool->transient_len();
    out->released = (uint32_t)p->pool->free_len();
    return HOLO_OK;
}
