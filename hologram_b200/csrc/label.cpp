#include "label.h"

#include <string.h>

#include "blake3.h"
#include "common.h"

void holo_label_from_digest(const uint8_t digest[32], uint8_t out[HOLO_LABEL_BYTES]) {
    static const char HEX[] = "0123456789abcdef";
    memcpy(out, "blake3:", 7);
    for (int i = 0; i < 32; ++i) {
        out[7 + 2 * i] = (uint8_t)HEX[digest[i] >> 4];
        out[7 + 2 * i + 1] = (uint8_t)HEX[digest[i] & 15];
    }
}

void holo_label_of_bytes(const uint8_t* data, size_t len, uint8_t out[HOLO_LABEL_BYTES]) {
    uint8_t d[32];
    holo_blake3(data, len, d);
    holo_label_from_digest(d, out);
}

void holo_label_derive(uint16_t opcode, const uint8_t* params, size_t params_len, const uint8_t* labels, size_t n_labels,
                       uint8_t out[HOLO_LABEL_BYTES]) {
    // the reference folds the pieces through a streaming hasher; hashing their concatenation is
    // the same digest
    std::vector<uint8_t> buf;
    buf.reserve(2 + params_len + n_labels * HOLO_LABEL_BYTES);
    buf.push_back((uint8_t)(opcode & 0xff));
    buf.push_back((uint8_t)(opcode >> 8));
    buf.insert(buf.end(), params, params + params_len);
    buf.insert(buf.end(), labels, labels + n_labels * HOLO_LABEL_BYTES);
    uint8_t d[32];
    holo_blake3(buf.data(), buf.size(), d);
    holo_label_from_digest(d, out);
}

// derive_label_boundary (address.rs:197-221): op label = address_bytes(opcode LE16 || params); every
// operand label is folded in order through the ordered product address_bytes(left digest || right
// digest) (compose.rs:154-164); with no operand the op label is composed with itself.
namespace {
bool label_digest(const uint8_t* label, uint8_t out[32]) {   // decode_blake3: "blake3:" + 64 lowercase hex digits
    if (memcmp(label, "blake3:", 7) != 0) return false;
    for (int i = 0; i < 32; ++i) {
        int v = 0;
        for (int h = 0; h < 2; ++h) {
            const uint8_t c = label[7 + 2 * i + h];
            int d;
            if (c >= '0' && c <= '9') d = c - '0';
            else if (c >= 'a' && c <= 'f') d = c - 'a' + 10;
            else return false;
            v = v * 16 + d;
        }
        out[i] = (uint8_t)v;
    }
    return true;
}
bool compose_ordered(const uint8_t* left, const uint8_t* right, uint8_t out[HOLO_LABEL_BYTES]) {
    uint8_t canon[64];
    if (!label_digest(left, canon) || !label_digest(right, canon + 32)) return false;
    holo_label_of_bytes(canon, 64, out);
    return true;
}
}  // namespace

bool holo_label_derive_boundary(uint16_t opcode, const uint8_t* params, size_t params_len, const uint8_t* labels, size_t n_labels,
                                uint8_t out[HOLO_LABEL_BYTES]) {
    std::vector<uint8_t> pre;
    pre.push_back((uint8_t)(opcode & 0xff));
    pre.push_back((uint8_t)(opcode >> 8));
    pre.insert(pre.end(), params, params + params_len);
    uint8_t acc[HOLO_LABEL_BYTES], op_label[HOLO_LABEL_BYTES];
    holo_label_of_bytes(pre.data(), pre.size(), op_label);
    memcpy(acc, op_label, HOLO_LABEL_BYTES);
    for (size_t i = 0; i < n_labels; ++i) {
        uint8_t next[HOLO_LABEL_BYTES];
        if (!compose_ordered(acc, labels + i * HOLO_LABEL_BYTES, next)) return false;
        memcpy(acc, next, HOLO_LABEL_BYTES);
    }
    if (n_labels == 0 && !compose_ordered(op_label, op_label, acc)) return false;
    memcpy(out, acc, HOLO_LABEL_BYTES);
    return true;
}

namespace {
// Little-endian parameter builder (kernel_call.rs:950-993).
struct Pb {
    HoloOpSignature* s;
    Pb& raw(const void* p, size_t n) {
        if (s->len + n <= sizeof s->params) {
            memcpy(s->params + s->len, p, n);
            s->len += (uint32_t)n;
        }
        return *this;
    }
    Pb& u8(uint8_t v) { return raw(&v, 1); }
    Pb& u16(uint16_t v) { return raw(&v, 2); }
    Pb& u32(uint32_t v) { return raw(&v, 4); }
    Pb& i32(int32_t v) { return raw(&v, 4); }
    Pb& u64(uint64_t v) { return raw(&v, 8); }
};
void p_matmul(Pb& b, const HoloMatMulCall& c) { b.u32(c.m).u32(c.k).u32(c.n).u8(c.dtype); }
void p_attn(Pb& b, uint32_t batch, uint32_t heads, uint32_t kv, uint32_t m, uint32_t past, uint32_t nnew, uint32_t d, uint32_t scale_bits,
            uint8_t dtype) {
    b.u32(batch).u32(heads).u32(kv).u32(m).u32(past).u32(nnew).u32(d).u32(scale_bits).u8(dtype);
}
bool present(const HoloBufferRef& r) { return r.slot != HOLO_NO_SLOT; }
}  // namespace

bool holo_op_signature(const HoloKernelCall& call, HoloOpSignature* sig) {
    *sig = HoloOpSignature();
    Pb b{sig};
    const auto& u = call.u;
    // the exact elementwise variants: opcode = wire discriminant - 1 (kernel_call.rs:1325-1368); Min, Max and
    // Equal are commutative (:1302-1315)
    if (holo_is_exact_unary(call.kind)) {
        sig->opcode = (uint16_t)(call.kind - 1);
        b.u64(u.unary.element_count).u16(u.unary.witt_bits).u8(u.unary.dtype);
        return true;
    }
    if (holo_is_exact_binary(call.kind)) {
        sig->opcode = (uint16_t)(call.kind - 1);
        sig->commutative = call.kind == HOLO_K_MIN || call.kind == HOLO_K_MAX || call.kind == HOLO_K_EQUAL;
        b.u64(u.binary.element_count).u16(u.binary.witt_bits).u8(u.binary.dtype);
        return true;
    }
    switch (call.kind) {
        // unary / binary: element_count u64, witt_bits u16, dtype u8 (p_unary / p_binary)
        case HOLO_K_SIGMOID: sig->opcode = 11; break;
        case HOLO_K_TANH: sig->opcode = 12; break;
        case HOLO_K_GELU: sig->opcode = 13; break;
        case HOLO_K_SILU: sig->opcode = 14; break;
        case HOLO_K_EXP: sig->opcode = 17; break;
        case HOLO_K_ERF: sig->opcode = 31; break;
        case HOLO_K_ADD: sig->opcode = 4; sig->commutative = true; break;
        case HOLO_K_MUL: sig->opcode = 6; sig->commutative = true; break;
        case HOLO_K_CONCAT: sig->opcode = 61; break;
        case HOLO_K_MATMUL: sig->opcode = 45; p_matmul(b, u.matmul); return true;
        case HOLO_K_MATMUL_ACTIVATION: sig->opcode = 105; p_matmul(b, u.matmul_activation.mm); b.u8(u.matmul_activation.act); return true;
        case HOLO_K_MATMUL_ADD: sig->opcode = 106; p_matmul(b, u.matmul_add.mm); return true;
        case HOLO_K_MATMUL_ADD_ACTIVATION: sig->opcode = 107; p_matmul(b, u.matmul_add_activation.mm); b.u8(u.matmul_add_activation.act); return true;
        case HOLO_K_LAYER_NORM: case HOLO_K_RMS_NORM: case HOLO_K_ADD_RMS_NORM: {
            const HoloNormCall& c = u.norm;
            sig->opcode = call.kind == HOLO_K_LAYER_NORM ? 49 : call.kind == HOLO_K_RMS_NORM ? 50 : 53;
            b.u32(c.batch).u32(c.feature).u32(c.channels).u32(c.num_groups).u64(c.epsilon_bits).u8(c.dtype).u8(present(c.residual) ? 1 : 0);
            return true;
        }
        case HOLO_K_RESHAPE: case HOLO_K_SLICE:
            sig->opcode = call.kind == HOLO_K_RESHAPE ? 59 : 62;
            b.u64(u.layout.element_count).u8(u.layout.dtype);
            return true;
        case HOLO_K_TRANSPOSE: {
            const HoloTransposeCall& c = u.transpose;
            sig->opcode = 60;
            b.u8(c.rank).u8(c.dtype);
            for (uint32_t i = 0; i < c.rank && i < 8; ++i) b.u32(c.dims[i]).u8(c.perm[i]);
            return true;
        }
        case HOLO_K_REDUCE_SUM: case HOLO_K_REDUCE_MEAN: case HOLO_K_REDUCE_PROD: case HOLO_K_REDUCE_MIN: case HOLO_K_REDUCE_MAX: {
            const HoloReduceCall& c = u.reduce;
            sig->opcode = (uint16_t)(call.kind - 1);   // ReduceSum..ReduceMax are opcodes 54..58 (kernel_call.rs:1380-1384)
            b.u64(c.element_count).u8(c.rank).u32(c.axes_mask).u8(c.keepdims ? 1 : 0).u8(c.dtype);
            for (uint32_t i = 0; i < c.rank && i < 8; ++i) b.u32(c.dims[i]);
            return true;
        }
        case HOLO_K_WHERE: sig->opcode = 77; b.u64(u.where.element_count).u8(u.where.dtype); return true;
        case HOLO_K_DEQUANT_ACTIVATION: {
            const HoloDequantActivationCall& c = u.dequant_activation;
            sig->opcode = 113;
            b.u64(c.element_count).u8(c.quant_dtype).u8(c.act).u8(c.dtype).u32(c.scale_bits).u32((uint32_t)c.zero_point);
            return true;
        }
        case HOLO_K_ATTENTION: {
            const HoloAttentionCall& c = u.attention;
            sig->opcode = 68;
            b.u32(c.batch).u32(c.heads).u32(c.seq).u32(c.head_dim).u32(c.kv_heads).u8(c.causal ? 1 : 0).u32(c.scale_bits).u8(c.dtype);
            return true;
        }
        case HOLO_K_EXPAND: {
            const HoloExpandCall& c = u.expand;
            sig->opcode = 71;
            b.u8(c.rank).u8(c.dtype);
            for (uint32_t i = 0; i < c.rank && i < 8; ++i) b.u32(c.in_dims[i]).u32(c.out_dims[i]);
            return true;
        }
        case HOLO_K_BROADCAST_BINARY: {
            const HoloBroadcastBinaryCall& c = u.broadcast_binary;
            sig->opcode = 112;
            b.u8(c.rank).u8(c.op).u8(c.small_is_lhs ? 1 : 0).u8(c.dtype);
            for (uint32_t i = 0; i < c.rank && i < 8; ++i) b.u32(c.in_dims[i]).u32(c.out_dims[i]);
            return true;
        }
        case HOLO_K_SOFTMAX: sig->opcode = 63; b.u32(u.softmax.batch).u32(u.softmax.feature).u8(u.softmax.dtype); return true;
        case HOLO_K_ROTARY: sig->opcode = 74; b.u64(u.rope.element_count).u32(u.rope.head_dim).u8(u.rope.dtype); return true;
        case HOLO_K_GATHER: {
            const HoloGatherCall& c = u.gather;
            sig->opcode = 114;
            b.u64(c.outer).u64(c.axis_dim).u64(c.inner).u64(c.num_indices).u8(c.idx_dtype).u8(c.dtype);
            return true;
        }
        case HOLO_K_CAST: sig->opcode = 115; b.u64(u.cast.element_count).u8(u.cast.src_dtype).u8(u.cast.dst_dtype); return true;
        case HOLO_K_DEQUANTIZE: {
            const HoloDequantizeCall& c = u.dequantize;
            sig->opcode = 104;
            b.u64(c.element_count).u32(c.channels).u32(c.inner).u8(c.quant_dtype).u8(c.dtype).u32(c.scale_bits).i32(c.zero_point)
                .u8(present(c.scales) ? 1 : 0);
            return true;
        }
        case HOLO_K_DECODE_ATTENTION: {
            const HoloDecodeAttentionCall& c = u.decode_attention;
            sig->opcode = 119;
            p_attn(b, c.batch, c.heads, c.kv_heads, c.q_rows, c.past_len, c.new_len, c.head_dim, c.scale_bits, c.dtype);
            return true;
        }
        case HOLO_K_KV_CACHE_WRITE: {
            const HoloKvCacheWriteCall& c = u.kv_cache_write;
            sig->opcode = 120;
            b.u32(c.planes).u32(c.bucket_rows).u32(c.new_rows).u32(c.row_bytes);
            return true;
        }
        case HOLO_K_DECODE_ATTENTION_VALID: {
            const HoloDecodeAttentionValidCall& c = u.decode_attention_valid;
            sig->opcode = 121;
            p_attn(b, c.batch, c.heads, c.kv_heads, c.q_rows, c.past_len, c.new_len, c.head_dim, c.scale_bits, c.dtype);
            return true;
        }
        case HOLO_K_MATMUL_DEQUANT_PLAIN: case HOLO_K_MATMUL_DEQUANT: case HOLO_K_MATMUL_DEQUANT_CODEBOOK: {
            // kernel_call.rs:1472-1500: the all-default form keeps tag 108 and the base bytes; activation quantization
            // or an epilogue take the extended tag 116 (the layout-only bq_omajor does not); a bound codebook takes
            // tag 117 and one more byte
            const HoloMatMulDequantCall& c = u.matmul_dequant;
            b.u32(c.m).u32(c.k).u32(c.n).u32(c.channels).u32(c.inner).u8(c.quant_dtype).u8(c.dtype).u32(c.scale_bits).i32(c.zero_point);
            if (present(c.codebook)) {
                sig->opcode = 117;
                b.u8(c.act_quant).u8(c.act).u8(present(c.residual) ? 1 : 0).u8(1);
            } else if (c.act_quant != 0 || c.act != 0 || present(c.residual)) {
                sig->opcode = 116;
                b.u8(c.act_quant).u8(c.act).u8(present(c.residual) ? 1 : 0);
            } else {
                sig->opcode = 108;
            }
            return true;
        }
        // extensions: the tag doubles as the opcode
        case HOLO_K_QUANTIZE_ROWS_I8: {
            const HoloQuantizeRowsI8Call& c = u.quantize_rows_i8;
            sig->opcode = HOLO_K_QUANTIZE_ROWS_I8;
            b.u64(c.rows).u32(c.row_len).u8(c.dtype);
            return true;
        }
        case HOLO_K_DECODE_ATTENTION_VALID_Q8: {
            const HoloDecodeAttentionValidQ8Call& c = u.decode_attention_valid_q8;
            sig->opcode = HOLO_K_DECODE_ATTENTION_VALID_Q8;
            p_attn(b, c.batch, c.heads, c.kv_heads, c.q_rows, c.past_len, c.new_len, c.head_dim, c.scale_bits, c.dtype);
            return true;
        }
        default: return false;   // AllReduce: its value depends on the other ranks, not on local labels
    }
    // the unary / binary group
    if (call.kind == HOLO_K_ADD || call.kind == HOLO_K_MUL || call.kind == HOLO_K_CONCAT)
        b.u64(u.binary.element_count).u16(u.binary.witt_bits).u8(u.binary.dtype);
    else
        b.u64(u.unary.element_count).u16(u.unary.witt_bits).u8(u.unary.dtype);
    return true;
}

bool holo_call_operands(const HoloKernelCall& call, std::vector<uint32_t>* inputs, uint32_t* output, bool residual_in_label) {
    inputs->clear();
    auto in = [&](const HoloBufferRef& r) {
        if (present(r)) inputs->push_back(r.slot);
    };
    const auto& u = call.u;
    if (holo_is_exact_unary(call.kind)) { in(u.unary.input); *output = u.unary.output.slot; return true; }
    if (holo_is_exact_binary(call.kind)) { in(u.binary.a); in(u.binary.b); *output = u.binary.output.slot; return true; }
    switch (call.kind) {
        case HOLO_K_SIGMOID: case HOLO_K_TANH: case HOLO_K_GELU: case HOLO_K_SILU: case HOLO_K_EXP: case HOLO_K_ERF:
            in(u.unary.input); *output = u.unary.output.slot; return true;
        case HOLO_K_ADD: case HOLO_K_MUL: case HOLO_K_CONCAT:
            in(u.binary.a); in(u.binary.b); *output = u.binary.output.slot; return true;
        case HOLO_K_MATMUL: in(u.matmul.a); in(u.matmul.b); *output = u.matmul.output.slot; return true;
        case HOLO_K_MATMUL_ACTIVATION:
            in(u.matmul_activation.mm.a); in(u.matmul_activation.mm.b); *output = u.matmul_activation.mm.output.slot; return true;
        case HOLO_K_MATMUL_ADD:
            in(u.matmul_add.mm.a); in(u.matmul_add.mm.b); in(u.matmul_add.residual); *output = u.matmul_add.mm.output.slot; return true;
        case HOLO_K_MATMUL_ADD_ACTIVATION: {
            const auto& c = u.matmul_add_activation;
            in(c.mm.a); in(c.mm.b); in(c.residual); *output = c.mm.output.slot; return true;
        }
        case HOLO_K_MATMUL_DEQUANT_PLAIN: case HOLO_K_MATMUL_DEQUANT: case HOLO_K_MATMUL_DEQUANT_CODEBOOK: {
            const auto& c = u.matmul_dequant;
            in(c.a); in(c.bq);
            if (c.channels > 0 && present(c.scales)) { in(c.scales); in(c.zero_points); }
            if (present(c.codebook)) in(c.codebook);   // after the quant operands, before the residual (kernel_call.rs:1589-1598)
            in(c.residual);
            *output = c.output.slot; return true;
        }
        case HOLO_K_LAYER_NORM: case HOLO_K_RMS_NORM: case HOLO_K_ADD_RMS_NORM:
            // the reference lists x, gamma, beta (kernel_call.rs:1612-1616), for AddRmsNorm too; on request the
            // residual operand is appended so that two sums over different residuals never share a label
            in(u.norm.x); in(u.norm.gamma); in(u.norm.beta);
            if (call.kind == HOLO_K_ADD_RMS_NORM && residual_in_label) in(u.norm.residual);
            *output = u.norm.output.slot; return true;
        case HOLO_K_RESHAPE: case HOLO_K_SLICE: in(u.layout.input); *output = u.layout.output.slot; return true;
        case HOLO_K_TRANSPOSE: in(u.transpose.input); *output = u.transpose.output.slot; return true;
        case HOLO_K_SOFTMAX: in(u.softmax.input); *output = u.softmax.output.slot; return true;
        case HOLO_K_REDUCE_SUM: case HOLO_K_REDUCE_MEAN: case HOLO_K_REDUCE_PROD: case HOLO_K_REDUCE_MIN: case HOLO_K_REDUCE_MAX:
            in(u.reduce.input); *output = u.reduce.output.slot; return true;
        case HOLO_K_WHERE: in(u.where.cond); in(u.where.a); in(u.where.b); *output = u.where.output.slot; return true;
        case HOLO_K_DEQUANT_ACTIVATION: in(u.dequant_activation.input); *output = u.dequant_activation.output.slot; return true;
        case HOLO_K_ATTENTION: in(u.attention.q); in(u.attention.k); in(u.attention.v); *output = u.attention.output.slot; return true;
        case HOLO_K_EXPAND: in(u.expand.input); *output = u.expand.output.slot; return true;
        case HOLO_K_BROADCAST_BINARY: in(u.broadcast_binary.small); in(u.broadcast_binary.other); *output = u.broadcast_binary.output.slot; return true;
        case HOLO_K_ROTARY: in(u.rope.x); in(u.rope.cos); in(u.rope.sin); *output = u.rope.output.slot; return true;
        case HOLO_K_GATHER: in(u.gather.data); in(u.gather.indices); *output = u.gather.output.slot; return true;
        case HOLO_K_CAST: in(u.cast.input); *output = u.cast.output.slot; return true;
        case HOLO_K_DEQUANTIZE:
            in(u.dequantize.input);
            if (present(u.dequantize.scales)) { in(u.dequantize.scales); in(u.dequantize.zero_points); }
            *output = u.dequantize.output.slot; return true;
        case HOLO_K_DECODE_ATTENTION: {
            const auto& c = u.decode_attention;
            in(c.q); in(c.k_past); in(c.v_past); in(c.k_new); in(c.v_new); in(c.mask); *output = c.output.slot; return true;
        }
        case HOLO_K_KV_CACHE_WRITE: {
            const auto& c = u.kv_cache_write;
            in(c.cache); in(c.new_rows_buf); in(c.pos); *output = c.output.slot; return true;
        }
        case HOLO_K_DECODE_ATTENTION_VALID: {
            const auto& c = u.decode_attention_valid;
            in(c.q); in(c.k_past); in(c.v_past); in(c.k_new); in(c.v_new); in(c.valid_len); *output = c.output.slot; return true;
        }
        case HOLO_K_DECODE_ATTENTION_VALID_Q8: {
            const auto& c = u.decode_attention_valid_q8;
            in(c.q); in(c.k_past); in(c.k_past_scales); in(c.v_past); in(c.v_past_scales); in(c.k_new); in(c.k_new_scales);
            in(c.v_new); in(c.v_new_scales); in(c.valid_len); *output = c.output.slot; return true;
        }
        default: return false;   // QuantizeRowsI8 has two outputs, AllReduce is not a function of local labels
    }
}
