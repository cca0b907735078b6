"""`.holo` archive writer for synthetic archives (the reference compiler cannot run without its
Rust toolchain). Byte layout follows crates/hologram-archive: framing writer.rs:185-226,
calls kernel_codec.rs:130-137 + put_* :569-873, ports writer.rs:246-263, constants
constant_codec.rs:66-95, weights writer.rs:388-440, exec plan writer.rs:325-336.
"""
import struct

import blake3

from . import kernel_call as kc

SEC_KERNEL_CALLS, SEC_WEIGHTS, SEC_INPUTS, SEC_OUTPUTS, SEC_CONSTANTS, SEC_EXEC_PLAN, SEC_EXTENSION = 1, 3, 9, 10, 11, 12, 14
FORMAT_VERSION = 3


def _buf(b):
    return struct.pack("<IQQ", b.slot, b.offset, b.length)


def _unary(c):
    return _buf(c.input) + _buf(c.output) + struct.pack("<QHB", c.element_count, c.witt_bits, c.dtype)


def _binary(c):
    return _buf(c.a) + _buf(c.b) + _buf(c.output) + struct.pack("<QHB", c.element_count, c.witt_bits, c.dtype)


def _matmul(c):
    return _buf(c.a) + _buf(c.b) + _buf(c.output) + struct.pack("<IIIBB", c.m, c.k, c.n, c.dtype, c.b_packed)


def encode_call(call):
    """`u16 discriminant + payload` for one KernelCall (kernel_codec.rs encode_one)."""
    k, u = call.kind, call.u
    out = struct.pack("<H", k)
    if k in (kc.K_SIGMOID, kc.K_TANH, kc.K_GELU, kc.K_SILU, kc.K_EXP, kc.K_ERF) + kc.EXACT_UNARY:
        return out + _unary(u.unary)
    if k in (kc.K_ADD, kc.K_MUL, kc.K_CONCAT) + kc.EXACT_BINARY:
        return out + _binary(u.binary)
    if k == kc.K_MATMUL:
        return out + _matmul(u.matmul)
    if k == kc.K_MATMUL_ACTIVATION:
        return out + _matmul(u.matmul_activation.mm) + struct.pack("<B", u.matmul_activation.act)
    if k == kc.K_MATMUL_ADD:
        return out + _matmul(u.matmul_add.mm) + _buf(u.matmul_add.residual)
    if k == kc.K_MATMUL_ADD_ACTIVATION:
        c = u.matmul_add_activation
        return out + _matmul(c.mm) + _buf(c.residual) + struct.pack("<B", c.act)
    if k in (kc.K_MATMUL_DEQUANT_PLAIN, kc.K_MATMUL_DEQUANT, kc.K_MATMUL_DEQUANT_CODEBOOK):
        c = u.matmul_dequant
        base = out + b"".join(_buf(b) for b in (c.a, c.bq, c.scales, c.zero_points, c.output)) + struct.pack(
            "<IIIIIBBII", c.m, c.k, c.n, c.channels, c.inner, c.quant_dtype, c.dtype, c.scale_bits, c.zero_point & 0xFFFFFFFF)
        if k == kc.K_MATMUL_DEQUANT_PLAIN:
            return base
        return base + struct.pack("<BBB", c.bq_omajor, c.act_quant, c.act) + _buf(c.residual) + (
            _buf(c.codebook) if k == kc.K_MATMUL_DEQUANT_CODEBOOK else b"")
    if k in (kc.K_LAYER_NORM, kc.K_RMS_NORM, kc.K_ADD_RMS_NORM):
        c = u.norm
        return out + _buf(c.x) + _buf(c.gamma) + _buf(c.beta) + _buf(c.residual) + _buf(c.output) + struct.pack(
            "<IIIIQB", c.batch, c.feature, c.channels, c.num_groups, c.epsilon_bits, c.dtype)
    if k == kc.K_ROTARY:
        c = u.rope
        return out + _buf(c.x) + _buf(c.cos) + _buf(c.sin) + _buf(c.output) + struct.pack("<IQB", c.head_dim, c.element_count, c.dtype)
    if k == kc.K_GATHER:
        c = u.gather
        return out + _buf(c.data) + _buf(c.indices) + _buf(c.output) + struct.pack(
            "<QQQQBB", c.outer, c.axis_dim, c.inner, c.num_indices, c.idx_dtype, c.dtype)
    if k == kc.K_CAST:
        c = u.cast
        return out + _buf(c.input) + _buf(c.output) + struct.pack("<QBB", c.element_count, c.src_dtype, c.dst_dtype)
    if k in (kc.K_REDUCE_SUM, kc.K_REDUCE_MEAN, kc.K_REDUCE_PROD, kc.K_REDUCE_MIN, kc.K_REDUCE_MAX):
        c = u.reduce
        return out + _buf(c.input) + _buf(c.output) + struct.pack("<QBIBB", c.element_count, c.rank, c.axes_mask, c.keepdims, c.dtype) + struct.pack(
            "<%dI" % c.rank, *list(c.dims)[:c.rank])
    if k == kc.K_WHERE:
        c = u.where
        return out + _buf(c.cond) + _buf(c.a) + _buf(c.b) + _buf(c.output) + struct.pack("<QB", c.element_count, c.dtype)
    if k == kc.K_DEQUANT_ACTIVATION:
        c = u.dequant_activation
        return out + _buf(c.input) + _buf(c.output) + struct.pack("<QBBBIi", c.element_count, c.quant_dtype, c.act, c.dtype, c.scale_bits, c.zero_point)
    if k == kc.K_ATTENTION:
        c = u.attention
        return out + _buf(c.q) + _buf(c.k) + _buf(c.v) + _buf(c.output) + struct.pack(
            "<IIIIIBIB", c.batch, c.heads, c.seq, c.head_dim, c.kv_heads, c.causal, c.scale_bits, c.dtype)
    if k == kc.K_EXPAND:
        c = u.expand
        return out + _buf(c.input) + _buf(c.output) + struct.pack("<B8I8IB", c.rank, *c.in_dims, *c.out_dims, c.dtype)
    if k == kc.K_BROADCAST_BINARY:
        c = u.broadcast_binary
        dims = b"".join(struct.pack("<II", c.in_dims[i], c.out_dims[i]) for i in range(c.rank))
        return out + _buf(c.small) + _buf(c.other) + _buf(c.output) + struct.pack("<BBBB", c.rank, c.op, c.small_is_lhs, c.dtype) + dims
    if k == kc.K_SOFTMAX:
        c = u.softmax
        return out + _buf(c.input) + _buf(c.output) + struct.pack("<IIB", c.batch, c.feature, c.dtype)
    if k == kc.K_TRANSPOSE:
        c = u.transpose
        return out + _buf(c.input) + _buf(c.output) + struct.pack("<B8I8BB", c.rank, *c.dims, *c.perm, c.dtype)
    if k in (kc.K_RESHAPE, kc.K_SLICE):
        c = u.layout
        return out + _buf(c.input) + _buf(c.output) + struct.pack("<QB", c.element_count, c.dtype)
    if k == kc.K_DEQUANTIZE:
        c = u.dequantize
        return out + _buf(c.input) + _buf(c.scales) + _buf(c.zero_points) + _buf(c.output) + struct.pack(
            "<QIIBBII", c.element_count, c.channels, c.inner, c.quant_dtype, c.dtype, c.scale_bits, c.zero_point & 0xFFFFFFFF)
    if k == kc.K_KV_CACHE_WRITE:
        c = u.kv_cache_write
        return out + _buf(c.cache) + _buf(c.new) + _buf(c.pos) + _buf(c.output) + struct.pack(
            "<IIII", c.planes, c.bucket_rows, c.new_rows, c.row_bytes)
    if k in (kc.K_DECODE_ATTENTION, kc.K_DECODE_ATTENTION_VALID):
        c = u.decode_attention if k == kc.K_DECODE_ATTENTION else u.decode_attention_valid
        sixth = c.mask if k == kc.K_DECODE_ATTENTION else c.valid_len
        bufs = b"".join(_buf(b) for b in (c.q, c.k_past, c.v_past, c.k_new, c.v_new, sixth, c.output))
        return out + bufs + struct.pack("<IIIIIIIIB", c.batch, c.heads, c.kv_heads, c.q_rows, c.past_len, c.new_len,
                                        c.head_dim, c.scale_bits, c.dtype)
    # extension discriminants (no counterpart in the reference codec)
    if k == kc.K_QUANTIZE_ROWS_I8:
        c = u.quantize_rows_i8
        return out + _buf(c.input) + _buf(c.codes) + _buf(c.scales) + struct.pack("<QIB", c.rows, c.row_len, c.dtype)
    if k == kc.K_DECODE_ATTENTION_VALID_Q8:
        c = u.decode_attention_valid_q8
        bufs = b"".join(_buf(b) for b in (c.q, c.k_past, c.k_past_scales, c.v_past, c.v_past_scales, c.k_new,
                                          c.k_new_scales, c.v_new, c.v_new_scales, c.valid_len, c.output))
        return out + bufs + struct.pack("<IIIIIIIIB", c.batch, c.heads, c.kv_heads, c.q_rows, c.past_len, c.new_len,
                                        c.head_dim, c.scale_bits, c.dtype)
    if k == kc.K_ROPE_QUANTIZE_ROWS_I8:
        c = u.rope_quantize
        return out + b"".join(_buf(b) for b in (c.x, c.cos, c.sin, c.rope_output, c.codes, c.scales)) + struct.pack(
            "<QIB", c.rows, c.row_len, c.dtype)
    if k == kc.K_ALL_REDUCE:
        c = u.all_reduce
        return out + _buf(c.buffer) + struct.pack("<QB", c.element_count, c.dtype)
    raise ValueError(f"no wire encoding for KernelCall kind {k}")


def encode_calls(calls):
    return struct.pack("<I", len(calls)) + b"".join(encode_call(c) for c in calls)


class Port:
    def __init__(self, name, slot, element_count, dtype, shape):
        self.name, self.slot, self.element_count, self.dtype, self.shape = name, slot, element_count, dtype, list(shape)


def encode_ports(ports):
    out = struct.pack("<I", len(ports))
    for p in ports:
        name = p.name.encode()
        out += struct.pack("<H", len(name)) + name + struct.pack("<IQBB", p.slot, p.element_count, p.dtype, len(p.shape))
        out += b"".join(struct.pack("<Q", d) for d in p.shape)
    return out


def fingerprint(body):
    return blake3.blake3(body, max_threads=blake3.blake3.AUTO).digest()


class HoloWriter:
    """Collects calls, ports and constants and frames them into a `.holo` image (HoloWriter::finish)."""

    def __init__(self):
        self.calls, self.inputs, self.outputs, self.exec_plan = [], [], [], []
        self.inline_constants, self.weight_constants, self.extensions = [], [], []

    def add_constant(self, slot, dtype, array_bytes, by_reference=None):
        body = bytes(array_bytes) if not isinstance(array_bytes, (bytes, bytearray, memoryview)) else array_bytes
        if by_reference is None:
            by_reference = len(body) > 256
        (self.weight_constants if by_reference else self.inline_constants).append((slot, dtype, body))

    def finish(self, weightless=False):
        """The archive image. `weightless`: constants stored by reference keep their fingerprints but the Weights
        section carries no bodies (they come from a weight provider at load, crates/hologram-exec/src/session.rs:417)."""
        weights, order, const = {}, [], struct.pack("<I", len(self.inline_constants) + len(self.weight_constants))
        for slot, dtype, body in self.inline_constants:
            const += struct.pack("<BIBI", 0, slot, dtype, len(body)) + bytes(body)
        for slot, dtype, body in self.weight_constants:
            fp = fingerprint(body)
            if fp not in weights:
                weights[fp] = body
                order.append(fp)
            const += struct.pack("<BIB", 1, slot, dtype) + fp
        self.weight_bodies = dict(weights)          # fingerprint -> body, what a weight provider serves
        if weightless:
            order = []
        wsec = [struct.pack("<I", len(order))]
        for fp in order:
            wsec += [fp, struct.pack("<Q", len(weights[fp])), weights[fp]]
        payloads = [(SEC_KERNEL_CALLS, [encode_calls(self.calls)]), (SEC_WEIGHTS, wsec)]
        if self.inputs:
            payloads.append((SEC_INPUTS, [encode_ports(self.inputs)]))
        if self.outputs:
            payloads.append((SEC_OUTPUTS, [encode_ports(self.outputs)]))
        if self.inline_constants or self.weight_constants:
            payloads.append((SEC_CONSTANTS, [const]))
        if self.exec_plan:
            ep = struct.pack("<I", len(self.exec_plan))
            for level in self.exec_plan:
                ep += struct.pack("<I", len(level)) + b"".join(struct.pack("<I", i) for i in level)
            payloads.append((SEC_EXEC_PLAN, [ep]))
        for key, body in self.extensions:
            k = key.encode()
            payloads.append((SEC_EXTENSION, [struct.pack("<H", len(k)) + k + body]))
        return assemble(payloads)


def assemble(payloads):
    """header || section table || payloads || 32-byte BLAKE3 footer (writer.rs:185-226)."""
    sizes = [sum(len(p) for p in parts) for _, parts in payloads]
    offset = 10 + 24 * len(payloads)
    head = b"HOLO" + struct.pack("<HHH", FORMAT_VERSION, 0, len(payloads))
    for (kind, _), size in zip(payloads, sizes):
        head += struct.pack("<B7xQQ", kind, offset, size)
        offset += size
    h = blake3.blake3(max_threads=blake3.blake3.AUTO)
    chunks = [head] + [p for _, parts in payloads for p in parts]
    for c in chunks:
        h.update(c)
    chunks.append(h.digest())
    return b"".join(bytes(c) if not isinstance(c, bytes) else c for c in chunks)
