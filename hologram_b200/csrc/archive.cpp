#include "archive.h"

#include <string.h>

#include <map>

#include "blake3.h"
#include "common.h"

namespace {

struct Reader {
    const uint8_t* p;
    uint64_t n, cur = 0;
    bool ok = true;
    bool need(uint64_t k) {
        if (!ok || k > n - cur) ok = false;   // cur <= n always; written so that a huge k cannot wrap
        return ok;
    }
    uint8_t u8() { return need(1) ? p[cur++] : 0; }
    uint16_t u16() {
        if (!need(2)) return 0;
        uint16_t v;
        memcpy(&v, p + cur, 2);
        cur += 2;
        return v;
    }
    uint32_t u32() {
        if (!need(4)) return 0;
        uint32_t v;
        memcpy(&v, p + cur, 4);
        cur += 4;
        return v;
    }
    uint64_t u64() {
        if (!need(8)) return 0;
        uint64_t v;
        memcpy(&v, p + cur, 8);
        cur += 8;
        return v;
    }
    HoloBufferRef buf() {  // put_buf, kernel_codec.rs:569-573
        HoloBufferRef b;
        b.slot = u32();
        b.offset = u64();
        b.length = u64();
        return b;
    }
};

void get_unary(Reader& r, HoloUnaryCall& c) {
    c.input = r.buf(); c.output = r.buf(); c.element_count = r.u64(); c.witt_bits = r.u16(); c.dtype = r.u8();
}
void get_binary(Reader& r, HoloBinaryCall& c) {
    c.a = r.buf(); c.b = r.buf(); c.output = r.buf(); c.element_count = r.u64(); c.witt_bits = r.u16(); c.dtype = r.u8();
}
void get_matmul(Reader& r, HoloMatMulCall& c) {
    c.a = r.buf(); c.b = r.buf(); c.output = r.buf(); c.m = r.u32(); c.k = r.u32(); c.n = r.u32(); c.dtype = r.u8(); c.b_packed = r.u8();
}

// decode_one for the served discriminants (crates/hologram-archive/src/decoder.rs:67+).
int32_t decode_call(Reader& r, HoloKernelCall* out) {
    memset(out, 0, sizeof *out);
    const uint16_t d = r.u16();
    out->kind = d;
    if (holo_is_exact_unary(d) || holo_is_exact_binary(d)) {
        if (holo_is_exact_unary(d)) get_unary(r, out->u.unary);
        else get_binary(r, out->u.binary);
        if (!r.ok) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated KernelCalls section");
        return HOLO_OK;
    }
    switch (d) {
        case HOLO_K_SIGMOID: case HOLO_K_TANH: case HOLO_K_GELU: case HOLO_K_SILU: case HOLO_K_EXP: case HOLO_K_ERF:
            get_unary(r, out->u.unary); break;
        case HOLO_K_ADD: case HOLO_K_MUL: case HOLO_K_CONCAT: get_binary(r, out->u.binary); break;
        case HOLO_K_TRANSPOSE: {
            HoloTransposeCall& c = out->u.transpose;
            c.input = r.buf(); c.output = r.buf(); c.rank = r.u8();
            for (int i = 0; i < 8; ++i) c.dims[i] = r.u32();
            for (int i = 0; i < 8; ++i) c.perm[i] = r.u8();
            c.dtype = r.u8();
            break;
        }
        case HOLO_K_MATMUL: get_matmul(r, out->u.matmul); break;
        case HOLO_K_MATMUL_ACTIVATION: get_matmul(r, out->u.matmul_activation.mm); out->u.matmul_activation.act = r.u8(); break;
        case HOLO_K_MATMUL_ADD: get_matmul(r, out->u.matmul_add.mm); out->u.matmul_add.residual = r.buf(); break;
        case HOLO_K_MATMUL_ADD_ACTIVATION:
            get_matmul(r, out->u.matmul_add_activation.mm); out->u.matmul_add_activation.residual = r.buf(); out->u.matmul_add_activation.act = r.u8();
            break;
        case HOLO_K_LAYER_NORM: case HOLO_K_RMS_NORM: case HOLO_K_ADD_RMS_NORM: {
            HoloNormCall& c = out->u.norm;
            c.x = r.buf(); c.gamma = r.buf(); c.beta = r.buf(); c.residual = r.buf(); c.output = r.buf();
            c.batch = r.u32(); c.feature = r.u32(); c.channels = r.u32(); c.num_groups = r.u32(); c.epsilon_bits = r.u64(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_REDUCE_SUM: case HOLO_K_REDUCE_MEAN: case HOLO_K_REDUCE_PROD: case HOLO_K_REDUCE_MIN: case HOLO_K_REDUCE_MAX: {
            HoloReduceCall& c = out->u.reduce;
            c.input = r.buf(); c.output = r.buf(); c.element_count = r.u64(); c.rank = r.u8(); c.axes_mask = r.u32();
            c.keepdims = r.u8(); c.dtype = r.u8();
            if (c.rank > 8) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: rank must be <= 8");
            for (uint32_t i = 0; i < c.rank; ++i) c.dims[i] = r.u32();
            break;
        }
        case HOLO_K_WHERE: {
            HoloWhereCall& c = out->u.where;
            c.cond = r.buf(); c.a = r.buf(); c.b = r.buf(); c.output = r.buf(); c.element_count = r.u64(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_DEQUANT_ACTIVATION: {
            HoloDequantActivationCall& c = out->u.dequant_activation;
            c.input = r.buf(); c.output = r.buf(); c.element_count = r.u64(); c.quant_dtype = r.u8(); c.act = r.u8(); c.dtype = r.u8();
            c.scale_bits = r.u32(); c.zero_point = (int32_t)r.u32();
            break;
        }
        case HOLO_K_ATTENTION: {
            HoloAttentionCall& c = out->u.attention;
            c.q = r.buf(); c.k = r.buf(); c.v = r.buf(); c.output = r.buf();
            c.batch = r.u32(); c.heads = r.u32(); c.seq = r.u32(); c.head_dim = r.u32(); c.kv_heads = r.u32();
            c.causal = r.u8(); c.scale_bits = r.u32(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_EXPAND: {
            HoloExpandCall& c = out->u.expand;
            c.input = r.buf(); c.output = r.buf(); c.rank = r.u8();
            for (int i = 0; i < 8; ++i) c.in_dims[i] = r.u32();
            for (int i = 0; i < 8; ++i) c.out_dims[i] = r.u32();
            c.dtype = r.u8();
            break;
        }
        case HOLO_K_BROADCAST_BINARY: {
            HoloBroadcastBinaryCall& c = out->u.broadcast_binary;
            c.small = r.buf(); c.other = r.buf(); c.output = r.buf();
            c.rank = r.u8(); c.op = r.u8(); c.small_is_lhs = r.u8(); c.dtype = r.u8();
            for (uint32_t i = 0; i < c.rank && i < 8; ++i) { c.in_dims[i] = r.u32(); c.out_dims[i] = r.u32(); }
            if (c.rank > 8) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: rank must be <= 8");
            break;
        }
        case HOLO_K_SOFTMAX: {
            HoloSoftmaxCall& c = out->u.softmax;
            c.input = r.buf(); c.output = r.buf(); c.batch = r.u32(); c.feature = r.u32(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_ROTARY: {
            HoloRoPECall& c = out->u.rope;
            c.x = r.buf(); c.cos = r.buf(); c.sin = r.buf(); c.output = r.buf(); c.head_dim = r.u32(); c.element_count = r.u64(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_GATHER: {
            HoloGatherCall& c = out->u.gather;
            c.data = r.buf(); c.indices = r.buf(); c.output = r.buf(); c.outer = r.u64(); c.axis_dim = r.u64(); c.inner = r.u64();
            c.num_indices = r.u64(); c.idx_dtype = r.u8(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_CAST: {
            HoloCastCall& c = out->u.cast;
            c.input = r.buf(); c.output = r.buf(); c.element_count = r.u64(); c.src_dtype = r.u8(); c.dst_dtype = r.u8();
            break;
        }
        case HOLO_K_RESHAPE: case HOLO_K_SLICE: {
            HoloLayoutCall& c = out->u.layout;
            c.input = r.buf(); c.output = r.buf(); c.element_count = r.u64(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_DEQUANTIZE: {
            HoloDequantizeCall& c = out->u.dequantize;
            c.input = r.buf(); c.scales = r.buf(); c.zero_points = r.buf(); c.output = r.buf(); c.element_count = r.u64();
            c.channels = r.u32(); c.inner = r.u32(); c.quant_dtype = r.u8(); c.dtype = r.u8(); c.scale_bits = r.u32(); c.zero_point = (int32_t)r.u32();
            break;
        }
        case HOLO_K_KV_CACHE_WRITE: {
            HoloKvCacheWriteCall& c = out->u.kv_cache_write;
            c.cache = r.buf(); c.new_rows_buf = r.buf(); c.pos = r.buf(); c.output = r.buf();
            c.planes = r.u32(); c.bucket_rows = r.u32(); c.new_rows = r.u32(); c.row_bytes = r.u32();
            break;
        }
        case HOLO_K_DECODE_ATTENTION: {
            HoloDecodeAttentionCall& c = out->u.decode_attention;
            c.q = r.buf(); c.k_past = r.buf(); c.v_past = r.buf(); c.k_new = r.buf(); c.v_new = r.buf(); c.mask = r.buf(); c.output = r.buf();
            c.batch = r.u32(); c.heads = r.u32(); c.kv_heads = r.u32(); c.q_rows = r.u32(); c.past_len = r.u32(); c.new_len = r.u32();
            c.head_dim = r.u32(); c.scale_bits = r.u32(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_DECODE_ATTENTION_VALID: {
            HoloDecodeAttentionValidCall& c = out->u.decode_attention_valid;
            c.q = r.buf(); c.k_past = r.buf(); c.v_past = r.buf(); c.k_new = r.buf(); c.v_new = r.buf(); c.valid_len = r.buf(); c.output = r.buf();
            c.batch = r.u32(); c.heads = r.u32(); c.kv_heads = r.u32(); c.q_rows = r.u32(); c.past_len = r.u32(); c.new_len = r.u32();
            c.head_dim = r.u32(); c.scale_bits = r.u32(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_QUANTIZE_ROWS_I8: {
            HoloQuantizeRowsI8Call& c = out->u.quantize_rows_i8;
            c.input = r.buf(); c.codes = r.buf(); c.scales = r.buf(); c.rows = r.u64(); c.row_len = r.u32(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_DECODE_ATTENTION_VALID_Q8: {
            HoloDecodeAttentionValidQ8Call& c = out->u.decode_attention_valid_q8;
            c.q = r.buf(); c.k_past = r.buf(); c.k_past_scales = r.buf(); c.v_past = r.buf(); c.v_past_scales = r.buf();
            c.k_new = r.buf(); c.k_new_scales = r.buf(); c.v_new = r.buf(); c.v_new_scales = r.buf(); c.valid_len = r.buf(); c.output = r.buf();
            c.batch = r.u32(); c.heads = r.u32(); c.kv_heads = r.u32(); c.q_rows = r.u32(); c.past_len = r.u32(); c.new_len = r.u32();
            c.head_dim = r.u32(); c.scale_bits = r.u32(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_MATMUL_DEQUANT_PLAIN: case HOLO_K_MATMUL_DEQUANT: case HOLO_K_MATMUL_DEQUANT_CODEBOOK: {
            HoloMatMulDequantCall& c = out->u.matmul_dequant;
            c.a = r.buf(); c.bq = r.buf(); c.scales = r.buf(); c.zero_points = r.buf(); c.output = r.buf();
            c.m = r.u32(); c.k = r.u32(); c.n = r.u32(); c.channels = r.u32(); c.inner = r.u32(); c.quant_dtype = r.u8(); c.dtype = r.u8();
            c.scale_bits = r.u32(); c.zero_point = (int32_t)r.u32();
            c.residual = c.codebook = HoloBufferRef{HOLO_NO_SLOT, 0, 0};
            if (d == HOLO_K_MATMUL_DEQUANT_PLAIN) break;   // D_MMDQ: every extended field at its default
            c.bq_omajor = r.u8(); c.act_quant = r.u8(); c.act = r.u8(); c.residual = r.buf();
            if (d == HOLO_K_MATMUL_DEQUANT_CODEBOOK) c.codebook = r.buf();
            break;
        }
        case HOLO_K_ROPE_QUANTIZE_ROWS_I8: {
            HoloRopeQuantizeCall& c = out->u.rope_quantize;
            c.x = r.buf(); c.cos = r.buf(); c.sin = r.buf(); c.rope_output = r.buf(); c.codes = r.buf(); c.scales = r.buf();
            c.rows = r.u64(); c.row_len = r.u32(); c.dtype = r.u8();
            break;
        }
        case HOLO_K_ALL_REDUCE: {
            HoloAllReduceCall& c = out->u.all_reduce;
            c.buffer = r.buf(); c.element_count = r.u64(); c.dtype = r.u8();
            break;
        }
        default:
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: kernel-call discriminant %u is not served by the B200 backend", d);
    }
    if (!r.ok) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated KernelCalls section");
    return HOLO_OK;
}

int32_t decode_ports(const uint8_t* p, uint64_t n, std::vector<HoloPort>* out) {
    Reader r{p, n};
    uint32_t count = r.u32();
    for (uint32_t i = 0; i < count && r.ok; ++i) {
        HoloPort port;
        uint16_t nl = r.u16();
        if (!r.need(nl)) break;
        port.name.assign((const char*)p + r.cur, nl);
        r.cur += nl;
        port.slot = r.u32();
        port.element_count = r.u64();
        port.dtype = r.u8();
        uint8_t rank = r.u8();
        for (uint8_t k = 0; k < rank; ++k) port.shape.push_back(r.u64());
        out->push_back(port);
    }
    if (!r.ok) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated port section");
    return HOLO_OK;
}

}  // namespace

int32_t holo_archive_parse(const uint8_t* data, uint64_t len, bool verify, HoloArchive* out, bool allow_missing_weights) {
    // header: magic, version in [2, 3], flags, section count (loader.rs:141-179)
    if (len < 10 + 32) return holo_fail(HOLO_ERR_INIT, "backend init failed: archive shorter than header + footer");
    if (memcmp(data, "HOLO", 4) != 0) return holo_fail(HOLO_ERR_INIT, "backend init failed: bad .holo magic");
    Reader h{data, len - 32};
    h.cur = 4;
    out->version = h.u16();
    if (out->version < 2 || out->version > 3) return holo_fail(HOLO_ERR_INIT, "backend init failed: unsupported .holo version %u", out->version);
    h.u16();  // flags
    const uint16_t nsec = h.u16();
    if (verify) {
        uint8_t digest[32];
        holo_blake3(data, len - 32, digest);
        if (memcmp(digest, data + len - 32, 32) != 0) return holo_fail(HOLO_ERR_INIT, "backend init failed: .holo footer checksum mismatch");
    }
    struct Sec { uint8_t kind; uint64_t off, n; };
    std::vector<Sec> secs;
    for (uint16_t i = 0; i < nsec; ++i) {
        Sec s;
        s.kind = h.u8();
        h.cur += 7;
        s.off = h.u64();
        s.n = h.u64();
        if (!h.ok || s.off > len - 32 || s.n > len - 32 - s.off) return holo_fail(HOLO_ERR_INIT, "backend init failed: section %u out of bounds", i);
        secs.push_back(s);
    }
    std::map<std::string, std::pair<const uint8_t*, uint64_t>> weights;  // fingerprint -> body
    bool have_calls = false;
    const Sec* constants = nullptr;
    for (const Sec& s : secs) {
        const uint8_t* p = data + s.off;
        switch (s.kind) {
            case 1: {  // KernelCalls: u32 count, then u16 discriminant + payload each
                Reader r{p, s.n};
                uint32_t count = r.u32();
                for (uint32_t i = 0; i < count; ++i) {
                    HoloKernelCall c;
                    HOLO_TRY(decode_call(r, &c));
                    out->calls.push_back(c);
                }
                have_calls = true;
                break;
            }
            case 3: {  // Weights: u32 count, {fp[32], len u64, bytes}
                Reader r{p, s.n};
                uint32_t count = r.u32();
                for (uint32_t i = 0; i < count; ++i) {
                    if (!r.need(40)) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated Weights section");
                    std::string fp((const char*)p + r.cur, 32);
                    r.cur += 32;
                    uint64_t blen = r.u64();
                    if (!r.need(blen)) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated weight body");
                    if (verify) {
                        uint8_t digest[32];
                        holo_blake3(p + r.cur, blen, digest);
                        if (memcmp(digest, fp.data(), 32) != 0) return holo_fail(HOLO_ERR_INIT, "backend init failed: weight fingerprint mismatch");
                    }
                    weights[fp] = {p + r.cur, blen};
                    r.cur += blen;
                }
                break;
            }
            case 9: HOLO_TRY(decode_ports(p, s.n, &out->inputs)); break;
            case 10: HOLO_TRY(decode_ports(p, s.n, &out->outputs)); break;
            case 11: constants = &s; break;
            case 12: {  // ExecPlan: levels u32, {n u32, idx u32 x n}
                Reader r{p, s.n};
                uint32_t levels = r.u32();
                for (uint32_t l = 0; l < levels && r.ok; ++l) {
                    uint32_t n = r.u32();
                    std::vector<uint32_t> lv;
                    for (uint32_t i = 0; i < n && r.ok; ++i) lv.push_back(r.u32());
                    out->exec_plan.push_back(lv);
                }
                if (!r.ok) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated ExecPlan section");
                break;
            }
            case 14: {  // Extension: key_len u16, key, bytes
                Reader r{p, s.n};
                uint16_t kl = r.u16();
                if (!r.need(kl)) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated Extension section");
                HoloExtension e;
                e.key.assign((const char*)p + r.cur, kl);
                e.bytes = p + r.cur + kl;
                e.len = s.n - r.cur - kl;
                out->extensions.push_back(e);
                break;
            }
            default: break;  // Schedule, registries, certificates, trace, metadata, warm start: not needed to execute
        }
    }
    if (!have_calls) return holo_fail(HOLO_ERR_INIT, "backend init failed: archive has no KernelCalls section");
    if (constants) {  // constant_codec.rs:66-95: tag 0 inline {slot, dtype, len u32, bytes}, tag 1 reference {slot, dtype, fp[32]}
        const uint8_t* p = data + constants->off;
        Reader r{p, constants->n};
        uint32_t count = r.u32();
        for (uint32_t i = 0; i < count; ++i) {
            HoloConstant c;
            uint8_t tag = r.u8();
            c.slot = r.u32();
            c.dtype = r.u8();
            if (tag == 0) {
                c.len = r.u32();
                if (!r.need(c.len)) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated inline constant");
                c.bytes = p + r.cur;
                r.cur += c.len;
            } else if (tag == 1) {
                if (!r.need(32)) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated constant reference");
                std::string fp((const char*)p + r.cur, 32);
                r.cur += 32;
                c.by_reference = true;
                memcpy(c.fingerprint, fp.data(), 32);
                auto it = weights.find(fp);
                if (it != weights.end()) {
                    c.bytes = it->second.first;
                    c.len = it->second.second;
                } else if (!allow_missing_weights) {
                    // a weightless archive loaded without a provider must fail loud: an empty body would be
                    // the label of empty content and every kernel downstream would read zeros (session.rs:669-686)
                    return holo_fail(HOLO_ERR_INIT, "backend init failed: constant references a weight that is not in the archive");
                }
            } else {
                return holo_fail(HOLO_ERR_INIT, "backend init failed: unknown constant tag %u", tag);
            }
            if (!r.ok) return holo_fail(HOLO_ERR_INIT, "backend init failed: truncated Constants section");
            out->constants.push_back(c);
        }
    }
    for (const auto& lv : out->exec_plan)
        for (uint32_t idx : lv)
            if (idx >= out->calls.size()) return holo_fail(HOLO_ERR_INIT, "backend init failed: ExecPlan index %u out of range", idx);
    // Slot numbers size the session's tables: a well-formed archive numbers its slots densely, so
    // none can exceed the number of buffer references it contains (12 per call at most, plus
    // ports and constants). A larger number is a malformed image, not a reason to allocate for it.
    const uint64_t slot_cap = 12ull * out->calls.size() + out->inputs.size() + out->outputs.size() + out->constants.size() + 64;
    auto slot_ok = [&](uint32_t slot) { return slot == HOLO_NO_SLOT || slot < slot_cap; };
    for (HoloKernelCall& c : out->calls) {
        HoloRefList refs;
        if (!holo_collect_refs(&c, &refs)) continue;
        for (int r = 0; r < refs.n; ++r)
            if (!slot_ok(refs.refs[r]->slot))
                return holo_fail(HOLO_ERR_INIT, "backend init failed: slot number %u is beyond what this archive can address", refs.refs[r]->slot);
    }
    for (const HoloPort& p : out->inputs)
        if (p.slot >= slot_cap) return holo_fail(HOLO_ERR_INIT, "backend init failed: slot number %u is beyond what this archive can address", p.slot);
    for (const HoloPort& p : out->outputs)
        if (p.slot >= slot_cap) return holo_fail(HOLO_ERR_INIT, "backend init failed: slot number %u is beyond what this archive can address", p.slot);
    for (const HoloConstant& k : out->constants)
        if (k.slot >= slot_cap) return holo_fail(HOLO_ERR_INIT, "backend init failed: slot number %u is beyond what this archive can address", k.slot);
    return HOLO_OK;
}
