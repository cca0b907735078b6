"""ctypes mirror of include/hologram_b200.h: the `KernelCall` tagged union and its payloads.

Names follow the reference (crates/hologram-compute/src/kernel_call.rs): BufferRef,
UnaryCall, MatMulCall, DecodeAttentionValidCall ... so tests read like the reference's own.
"""
import ctypes as C

# dtype tags (crates/hologram-types/src/dtype_id.rs:51-74)
DTYPE_BOOL, DTYPE_U8, DTYPE_I8, DTYPE_U64, DTYPE_I32, DTYPE_I64 = 0, 1, 2, 3, 4, 5
DTYPE_F16, DTYPE_BF16, DTYPE_F32, DTYPE_F64 = 6, 7, 8, 9
DTYPE_I4 = 10     # two signed nibbles per byte, low nibble first

# lut_act ids (kernel_call.rs:877-885)
LUT_SIGMOID, LUT_TANH, LUT_GELU, LUT_SILU, LUT_EXP, LUT_ERF = 0, 1, 2, 3, 4, 5
LUT_NAMES = {LUT_SIGMOID: "sigmoid", LUT_TANH: "tanh", LUT_GELU: "gelu", LUT_SILU: "silu", LUT_EXP: "exp", LUT_ERF: "erf"}

# fused_activation ids (kernel_call.rs:861-870)
FUSED_RELU, FUSED_GELU, FUSED_SILU, FUSED_SIGMOID, FUSED_TANH, FUSED_EXP = 1, 2, 3, 4, 5, 8

# variant tags = archive wire discriminants (crates/hologram-archive/src/kernel_codec.rs:19-128)
K_ADD, K_MUL = 5, 7
# exact elementwise variants (one IEEE operation per element)
K_NEG, K_RELU, K_SQRT, K_RECIPROCAL, K_CEIL, K_FLOOR, K_ROUND, K_IS_NAN, K_SIGN, K_ABS = 1, 11, 21, 22, 29, 30, 31, 33, 34, 35
K_SUB, K_DIV, K_MOD, K_MIN, K_MAX, K_EQUAL, K_LESS, K_LESS_OR_EQUAL, K_GREATER, K_GREATER_OR_EQUAL = 6, 36, 38, 39, 40, 41, 42, 43, 44, 45
EXACT_UNARY = (K_NEG, K_RELU, K_SQRT, K_RECIPROCAL, K_CEIL, K_FLOOR, K_ROUND, K_IS_NAN, K_SIGN, K_ABS)
EXACT_BINARY = (K_SUB, K_DIV, K_MOD, K_MIN, K_MAX, K_EQUAL, K_LESS, K_LESS_OR_EQUAL, K_GREATER, K_GREATER_OR_EQUAL)
K_SIGMOID, K_TANH, K_GELU, K_SILU, K_EXP, K_ERF = 12, 13, 14, 15, 18, 32
K_MATMUL, K_RMS_NORM, K_RESHAPE, K_ROTARY = 46, 51, 60, 75
K_LAYER_NORM, K_EXPAND, K_BROADCAST_BINARY, K_ATTENTION, K_DEQUANT_ACTIVATION, K_WHERE = 50, 72, 112, 69, 113, 78
BROADCAST_ADD, BROADCAST_SUB, BROADCAST_MUL = 0, 1, 2
K_REDUCE_SUM, K_REDUCE_MEAN, K_REDUCE_PROD, K_REDUCE_MIN, K_REDUCE_MAX = 55, 56, 57, 58, 59
K_ADD_RMS_NORM, K_TRANSPOSE, K_CONCAT, K_SLICE, K_SOFTMAX = 54, 61, 62, 63, 64
K_DECODE_ATTENTION = 119
K_MATMUL_DEQUANT = 116
K_MATMUL_DEQUANT_PLAIN = 111      # the all-default wire form ([k,n] weight, f32 activations)
K_MATMUL_ADD_ACTIVATION = 108
K_MATMUL_DEQUANT_CODEBOOK = 117   # the same call with a codebook operand bound (E8 codebook weights)
DTYPE_E8CB = 11
K_DEQUANTIZE, K_MATMUL_ACTIVATION, K_MATMUL_ADD = 105, 106, 107
K_GATHER, K_CAST, K_KV_CACHE_WRITE, K_DECODE_ATTENTION_VALID = 114, 115, 120, 121
K_QUANTIZE_ROWS_I8, K_DECODE_ATTENTION_VALID_Q8, K_ALL_REDUCE = 0x8001, 0x8002, 0x8003
K_ROPE_QUANTIZE_ROWS_I8 = 0x8004
LUT_KIND = {LUT_SIGMOID: K_SIGMOID, LUT_TANH: K_TANH, LUT_GELU: K_GELU, LUT_SILU: K_SILU, LUT_EXP: K_EXP, LUT_ERF: K_ERF}

NO_SLOT = 0xFFFFFFFF

# status codes (crates/hologram-compute/src/error.rs:6-20)
OK, ERR_SLOT_OUT_OF_RANGE, ERR_SHAPE_MISMATCH, ERR_UNSUPPORTED_OP, ERR_INIT, ERR_DISPATCH = 0, -1, -2, -3, -4, -5


class BufferRef(C.Structure):
    _fields_ = [("slot", C.c_uint32), ("offset", C.c_uint64), ("length", C.c_uint64)]


def rb(slot, offset=0, length=0):
    """BufferRef over a whole slot (the reference tests' `rb` helper, tests/lut.rs:51-57)."""
    return BufferRef(slot, offset, length)


NONE = BufferRef(NO_SLOT, 0, 0)


class UnaryCall(C.Structure):
    _fields_ = [("input", BufferRef), ("output", BufferRef), ("element_count", C.c_uint64),
                ("witt_bits", C.c_uint16), ("dtype", C.c_uint8)]


class BinaryCall(C.Structure):
    _fields_ = [("a", BufferRef), ("b", BufferRef), ("output", BufferRef), ("element_count", C.c_uint64),
                ("witt_bits", C.c_uint16), ("dtype", C.c_uint8)]


class MatMulCall(C.Structure):
    _fields_ = [("a", BufferRef), ("b", BufferRef), ("output", BufferRef), ("m", C.c_uint32), ("k", C.c_uint32),
                ("n", C.c_uint32), ("dtype", C.c_uint8), ("b_packed", C.c_uint8)]


class MatMulActivationCall(C.Structure):
    _fields_ = [("mm", MatMulCall), ("act", C.c_uint8)]


class MatMulAddCall(C.Structure):
    _fields_ = [("mm", MatMulCall), ("residual", BufferRef)]


class MatMulAddActivationCall(C.Structure):
    """kernel_call.rs:913-929: out = act(A . B + residual)."""
    _fields_ = [("mm", MatMulCall), ("residual", BufferRef), ("act", C.c_uint8)]


class MatMulDequantCall(C.Structure):
    """kernel_call.rs:152-213 (wire forms 111 / 116 / 117). Served: output-major W8A8 (bq_omajor=1, act_quant=1) over
    i8 / i4 / e8cb weights, and the [k,n] form with f32 activations (bq_omajor=0, act_quant=0) over i8 / u8 / i4."""
    _fields_ = [("a", BufferRef), ("bq", BufferRef), ("scales", BufferRef), ("zero_points", BufferRef), ("output", BufferRef),
                ("m", C.c_uint32), ("k", C.c_uint32), ("n", C.c_uint32), ("channels", C.c_uint32), ("inner", C.c_uint32),
                ("quant_dtype", C.c_uint8), ("dtype", C.c_uint8), ("scale_bits", C.c_uint32), ("zero_point", C.c_int32),
                ("bq_omajor", C.c_uint8), ("act_quant", C.c_uint8), ("act", C.c_uint8), ("residual", BufferRef), ("codebook", BufferRef)]

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        if len(args) < 19 and "codebook" not in kw:
            self.codebook = NONE


class NormCall(C.Structure):
    _fields_ = [("x", BufferRef), ("gamma", BufferRef), ("beta", BufferRef), ("residual", BufferRef),
                ("output", BufferRef), ("batch", C.c_uint32), ("feature", C.c_uint32), ("channels", C.c_uint32),
                ("num_groups", C.c_uint32), ("epsilon_bits", C.c_uint64), ("dtype", C.c_uint8)]


class RoPECall(C.Structure):
    _fields_ = [("x", BufferRef), ("cos", BufferRef), ("sin", BufferRef), ("output", BufferRef),
                ("head_dim", C.c_uint32), ("element_count", C.c_uint64), ("dtype", C.c_uint8)]


class GatherCall(C.Structure):
    _fields_ = [("data", BufferRef), ("indices", BufferRef), ("output", BufferRef), ("outer", C.c_uint64),
                ("axis_dim", C.c_uint64), ("inner", C.c_uint64), ("num_indices", C.c_uint64),
                ("idx_dtype", C.c_uint8), ("dtype", C.c_uint8)]


class CastCall(C.Structure):
    _fields_ = [("input", BufferRef), ("output", BufferRef), ("element_count", C.c_uint64),
                ("src_dtype", C.c_uint8), ("dst_dtype", C.c_uint8)]


class LayoutCall(C.Structure):
    _fields_ = [("input", BufferRef), ("output", BufferRef), ("element_count", C.c_uint64), ("dtype", C.c_uint8)]


class SoftmaxCall(C.Structure):
    _fields_ = [("input", BufferRef), ("output", BufferRef), ("batch", C.c_uint32), ("feature", C.c_uint32), ("dtype", C.c_uint8)]


class WhereCall(C.Structure):
    """kernel_call.rs:761-769: out[i] = cond[i] != 0 ? a[i] : b[i]; one condition byte per element."""
    _fields_ = [("cond", BufferRef), ("a", BufferRef), ("b", BufferRef), ("output", BufferRef), ("element_count", C.c_uint64),
                ("dtype", C.c_uint8)]


class DequantActivationCall(C.Structure):
    """kernel_call.rs:265-290: out = act((q - zero_point) * scale), i8 / u8 / i4 in, f32 out; act is a LUT_* id."""
    _fields_ = [("input", BufferRef), ("output", BufferRef), ("element_count", C.c_uint64), ("quant_dtype", C.c_uint8),
                ("act", C.c_uint8), ("dtype", C.c_uint8), ("scale_bits", C.c_uint32), ("zero_point", C.c_int32)]


class AttentionCall(C.Structure):
    """kernel_call.rs:575-594: q [b, heads, seq, d], k / v [b, kv_heads, seq, d]; causal: row i sees keys j <= i."""
    _fields_ = [("q", BufferRef), ("k", BufferRef), ("v", BufferRef), ("output", BufferRef), ("batch", C.c_uint32),
                ("heads", C.c_uint32), ("seq", C.c_uint32), ("head_dim", C.c_uint32), ("kv_heads", C.c_uint32),
                ("causal", C.c_uint8), ("scale_bits", C.c_uint32), ("dtype", C.c_uint8)]


class ReduceCall(C.Structure):
    """kernel_call.rs:461-477: fold the axes set in axes_mask (0 = all); keepdims layout."""
    _fields_ = [("input", BufferRef), ("output", BufferRef), ("element_count", C.c_uint64), ("rank", C.c_uint8),
                ("dims", C.c_uint32 * 8), ("axes_mask", C.c_uint32), ("keepdims", C.c_uint8), ("dtype", C.c_uint8)]

    @classmethod
    def make(cls, inp, out, dims, axes_mask, dtype, keepdims=True):
        c = cls()
        c.input, c.output, c.rank, c.axes_mask, c.keepdims, c.dtype = inp, out, len(dims), axes_mask, int(keepdims), dtype
        n = 1
        for i, d in enumerate(dims):
            c.dims[i] = d
            n *= d
        c.element_count = n
        return c


class ExpandCall(C.Structure):
    """kernel_call.rs:539-547: an axis with in_dims[i] == 1 reads index 0, the others map 1:1."""
    _fields_ = [("input", BufferRef), ("output", BufferRef), ("rank", C.c_uint8), ("in_dims", C.c_uint32 * 8),
                ("out_dims", C.c_uint32 * 8), ("dtype", C.c_uint8)]

    @classmethod
    def make(cls, inp, out, in_dims, out_dims, dtype):
        c = cls()
        c.input, c.output, c.rank, c.dtype = inp, out, len(out_dims), dtype
        for i, (a, b) in enumerate(zip(in_dims, out_dims)):
            c.in_dims[i], c.out_dims[i] = a, b
        return c


class BroadcastBinaryCall(C.Structure):
    """kernel_call.rs:292-317: out[o] = op(small[bcast(o)], other[o]) (swapped when small_is_lhs is 0)."""
    _fields_ = [("small", BufferRef), ("other", BufferRef), ("output", BufferRef), ("rank", C.c_uint8),
                ("in_dims", C.c_uint32 * 8), ("out_dims", C.c_uint32 * 8), ("op", C.c_uint8), ("small_is_lhs", C.c_uint8),
                ("dtype", C.c_uint8)]

    @classmethod
    def make(cls, small, other, out, in_dims, out_dims, op, small_is_lhs, dtype):
        c = cls()
        c.small, c.other, c.output, c.rank = small, other, out, len(out_dims)
        c.op, c.small_is_lhs, c.dtype = op, int(small_is_lhs), dtype
        for i, (a, b) in enumerate(zip(in_dims, out_dims)):
            c.in_dims[i], c.out_dims[i] = a, b
        return c


class TransposeCall(C.Structure):
    """kernel_call.rs:491-499: output axis i is input axis perm[i]."""
    _fields_ = [("input", BufferRef), ("output", BufferRef), ("rank", C.c_uint8), ("dims", C.c_uint32 * 8),
                ("perm", C.c_uint8 * 8), ("dtype", C.c_uint8)]

    @classmethod
    def make(cls, inp, out, dims, perm, dtype):
        c = cls()
        c.input, c.output, c.rank, c.dtype = inp, out, len(dims), dtype
        for i, (d, p) in enumerate(zip(dims, perm)):
            c.dims[i], c.perm[i] = d, p
        return c


class DequantizeCall(C.Structure):
    _fields_ = [("input", BufferRef), ("scales", BufferRef), ("zero_points", BufferRef), ("output", BufferRef),
                ("element_count", C.c_uint64), ("channels", C.c_uint32), ("inner", C.c_uint32),
                ("quant_dtype", C.c_uint8), ("dtype", C.c_uint8), ("scale_bits", C.c_uint32),
                ("zero_point", C.c_int32)]


class KvCacheWriteCall(C.Structure):
    _fields_ = [("cache", BufferRef), ("new", BufferRef), ("pos", BufferRef), ("output", BufferRef),
                ("planes", C.c_uint32), ("bucket_rows", C.c_uint32), ("new_rows", C.c_uint32),
                ("row_bytes", C.c_uint32)]


class DecodeAttentionValidCall(C.Structure):
    _fields_ = [("q", BufferRef), ("k_past", BufferRef), ("v_past", BufferRef), ("k_new", BufferRef),
                ("v_new", BufferRef), ("valid_len", BufferRef), ("output", BufferRef), ("batch", C.c_uint32),
                ("heads", C.c_uint32), ("kv_heads", C.c_uint32), ("q_rows", C.c_uint32), ("past_len", C.c_uint32),
                ("new_len", C.c_uint32), ("head_dim", C.c_uint32), ("scale_bits", C.c_uint32), ("dtype", C.c_uint8)]


class DecodeAttentionCall(C.Structure):
    """The additive-mask form (kernel_call.rs:632-655): mask is f32 [q_rows, past_len + new_len]."""
    _fields_ = [("q", BufferRef), ("k_past", BufferRef), ("v_past", BufferRef), ("k_new", BufferRef),
                ("v_new", BufferRef), ("mask", BufferRef), ("output", BufferRef), ("batch", C.c_uint32),
                ("heads", C.c_uint32), ("kv_heads", C.c_uint32), ("q_rows", C.c_uint32), ("past_len", C.c_uint32),
                ("new_len", C.c_uint32), ("head_dim", C.c_uint32), ("scale_bits", C.c_uint32), ("dtype", C.c_uint8)]


class QuantizeRowsI8Call(C.Structure):
    _fields_ = [("input", BufferRef), ("codes", BufferRef), ("scales", BufferRef), ("rows", C.c_uint64),
                ("row_len", C.c_uint32), ("dtype", C.c_uint8)]


class DecodeAttentionValidQ8Call(C.Structure):
    _fields_ = [("q", BufferRef), ("k_past", BufferRef), ("k_past_scales", BufferRef), ("v_past", BufferRef),
                ("v_past_scales", BufferRef), ("k_new", BufferRef), ("k_new_scales", BufferRef), ("v_new", BufferRef),
                ("v_new_scales", BufferRef), ("valid_len", BufferRef), ("output", BufferRef), ("batch", C.c_uint32),
                ("heads", C.c_uint32), ("kv_heads", C.c_uint32), ("q_rows", C.c_uint32), ("past_len", C.c_uint32),
                ("new_len", C.c_uint32), ("head_dim", C.c_uint32), ("scale_bits", C.c_uint32), ("dtype", C.c_uint8)]


class RopeQuantizeCall(C.Structure):
    """Extension: RotaryEmbedding then QuantizeRowsI8 of its result, one row = one head."""
    _fields_ = [("x", BufferRef), ("cos", BufferRef), ("sin", BufferRef), ("rope_output", BufferRef), ("codes", BufferRef),
                ("scales", BufferRef), ("rows", C.c_uint64), ("row_len", C.c_uint32), ("dtype", C.c_uint8)]


class AllReduceCall(C.Structure):
    _fields_ = [("buffer", BufferRef), ("element_count", C.c_uint64), ("dtype", C.c_uint8)]


class _Payload(C.Union):
    _fields_ = [("unary", UnaryCall), ("binary", BinaryCall), ("matmul", MatMulCall),
                ("matmul_activation", MatMulActivationCall), ("matmul_add", MatMulAddCall), ("matmul_add_activation", MatMulAddActivationCall), ("matmul_dequant", MatMulDequantCall), ("norm", NormCall),
                ("rope", RoPECall), ("gather", GatherCall), ("cast", CastCall), ("layout", LayoutCall),
                ("transpose", TransposeCall), ("softmax", SoftmaxCall), ("expand", ExpandCall), ("reduce", ReduceCall), ("attention", AttentionCall), ("dequant_activation", DequantActivationCall), ("where", WhereCall), ("broadcast_binary", BroadcastBinaryCall), ("dequantize", DequantizeCall), ("kv_cache_write", KvCacheWriteCall),
                ("decode_attention", DecodeAttentionCall),
                ("decode_attention_valid", DecodeAttentionValidCall), ("quantize_rows_i8", QuantizeRowsI8Call),
                ("decode_attention_valid_q8", DecodeAttentionValidQ8Call), ("all_reduce", AllReduceCall),
                ("rope_quantize", RopeQuantizeCall)]


class KernelCall(C.Structure):
    """`enum KernelCall` (kernel_call.rs:1146-1276) as tag + union."""
    _fields_ = [("kind", C.c_uint16), ("u", _Payload)]

    _FIELD = {}

    @classmethod
    def of(cls, kind, payload):
        kc = cls()
        kc.kind = kind
        setattr(kc.u, cls._FIELD[type(payload)], payload)
        return kc

    @classmethod
    def Elementwise(cls, kind, c):
        """Any of EXACT_UNARY (UnaryCall) or EXACT_BINARY (BinaryCall), by wire discriminant."""
        assert kind in EXACT_UNARY + EXACT_BINARY
        return cls.of(kind, c)

    # constructors named after the reference variants
    @classmethod
    def Sigmoid(cls, c): return cls.of(K_SIGMOID, c)
    @classmethod
    def Tanh(cls, c): return cls.of(K_TANH, c)
    @classmethod
    def Gelu(cls, c): return cls.of(K_GELU, c)
    @classmethod
    def Silu(cls, c): return cls.of(K_SILU, c)
    @classmethod
    def Exp(cls, c): return cls.of(K_EXP, c)
    @classmethod
    def Erf(cls, c): return cls.of(K_ERF, c)
    @classmethod
    def Add(cls, c): return cls.of(K_ADD, c)
    @classmethod
    def Mul(cls, c): return cls.of(K_MUL, c)
    @classmethod
    def MatMul(cls, c): return cls.of(K_MATMUL, c)
    @classmethod
    def MatMulActivation(cls, c): return cls.of(K_MATMUL_ACTIVATION, c)
    @classmethod
    def MatMulAdd(cls, c): return cls.of(K_MATMUL_ADD, c)
    @classmethod
    def MatMulAddActivation(cls, c): return cls.of(K_MATMUL_ADD_ACTIVATION, c)
    @classmethod
    def MatMulDequant(cls, c):
        # the wire form follows the call (kernel_codec.rs:525-544): a codebook takes 117, any extended field 116, else 111
        if c.codebook.slot != NO_SLOT:
            return cls.of(K_MATMUL_DEQUANT_CODEBOOK, c)
        extended = c.bq_omajor or c.act_quant or c.act or c.residual.slot != NO_SLOT
        return cls.of(K_MATMUL_DEQUANT if extended else K_MATMUL_DEQUANT_PLAIN, c)
    @classmethod
    def RmsNorm(cls, c): return cls.of(K_RMS_NORM, c)
    @classmethod
    def LayerNorm(cls, c): return cls.of(K_LAYER_NORM, c)
    @classmethod
    def AddRmsNorm(cls, c): return cls.of(K_ADD_RMS_NORM, c)
    @classmethod
    def Softmax(cls, c): return cls.of(K_SOFTMAX, c)
    @classmethod
    def Expand(cls, c): return cls.of(K_EXPAND, c)
    @classmethod
    def Attention(cls, c): return cls.of(K_ATTENTION, c)
    @classmethod
    def DequantActivation(cls, c): return cls.of(K_DEQUANT_ACTIVATION, c)
    @classmethod
    def Where(cls, c): return cls.of(K_WHERE, c)
    @classmethod
    def ReduceSum(cls, c): return cls.of(K_REDUCE_SUM, c)
    @classmethod
    def ReduceMean(cls, c): return cls.of(K_REDUCE_MEAN, c)
    @classmethod
    def ReduceProd(cls, c): return cls.of(K_REDUCE_PROD, c)
    @classmethod
    def ReduceMin(cls, c): return cls.of(K_REDUCE_MIN, c)
    @classmethod
    def ReduceMax(cls, c): return cls.of(K_REDUCE_MAX, c)
    @classmethod
    def BroadcastBinary(cls, c): return cls.of(K_BROADCAST_BINARY, c)
    @classmethod
    def Transpose(cls, c): return cls.of(K_TRANSPOSE, c)
    @classmethod
    def Concat(cls, c): return cls.of(K_CONCAT, c)
    @classmethod
    def Slice(cls, c): return cls.of(K_SLICE, c)
    @classmethod
    def RotaryEmbedding(cls, c): return cls.of(K_ROTARY, c)
    @classmethod
    def Gather(cls, c): return cls.of(K_GATHER, c)
    @classmethod
    def Cast(cls, c): return cls.of(K_CAST, c)
    @classmethod
    def Reshape(cls, c): return cls.of(K_RESHAPE, c)
    @classmethod
    def Dequantize(cls, c): return cls.of(K_DEQUANTIZE, c)
    @classmethod
    def KvCacheWrite(cls, c): return cls.of(K_KV_CACHE_WRITE, c)
    @classmethod
    def DecodeAttention(cls, c): return cls.of(K_DECODE_ATTENTION, c)
    @classmethod
    def DecodeAttentionValid(cls, c): return cls.of(K_DECODE_ATTENTION_VALID, c)
    @classmethod
    def QuantizeRowsI8(cls, c): return cls.of(K_QUANTIZE_ROWS_I8, c)
    @classmethod
    def DecodeAttentionValidQ8(cls, c): return cls.of(K_DECODE_ATTENTION_VALID_Q8, c)
    @classmethod
    def AllReduce(cls, c): return cls.of(K_ALL_REDUCE, c)
    @classmethod
    def RopeQuantizeRowsI8(cls, c): return cls.of(K_ROPE_QUANTIZE_ROWS_I8, c)


KernelCall._FIELD = {
    UnaryCall: "unary", BinaryCall: "binary", MatMulCall: "matmul", MatMulActivationCall: "matmul_activation",
    MatMulAddCall: "matmul_add", MatMulAddActivationCall: "matmul_add_activation", MatMulDequantCall: "matmul_dequant", NormCall: "norm", RoPECall: "rope", GatherCall: "gather", CastCall: "cast",
    LayoutCall: "layout", TransposeCall: "transpose", SoftmaxCall: "softmax", ExpandCall: "expand", ReduceCall: "reduce", AttentionCall: "attention", DequantActivationCall: "dequant_activation", WhereCall: "where", BroadcastBinaryCall: "broadcast_binary", DequantizeCall: "dequantize", KvCacheWriteCall: "kv_cache_write",
    DecodeAttentionCall: "decode_attention", DecodeAttentionValidCall: "decode_attention_valid", QuantizeRowsI8Call: "quantize_rows_i8",
    DecodeAttentionValidQ8Call: "decode_attention_valid_q8", AllReduceCall: "all_reduce", RopeQuantizeCall: "rope_quantize",
}


class HostSlot(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("bytes", C.c_uint64)]


def lut_call(act, c):
    """KernelCall for LUT activation id `act` over UnaryCall `c`."""
    return KernelCall.of(LUT_KIND[act], c)
