/*
 * hologram_b200.h — C ABI of the B200 (sm_100a) backend for hologram's tensor engine.
 *
 * The library is a drop-in for ONE boundary of the reference: `Backend::dispatch(&KernelCall,
 * &mut Workspace)` (crates/hologram-compute/src/backend.rs:8-15). A Rust `impl Backend`
 * forwards each call through `holo_b200_dispatch`; everything above that boundary (compiler,
 * archive, session walk) stays the reference's.
 *
 * Conventions follow crates/hologram-ffi (src/lib.rs:48-92): every function returns an
 * int32_t status (0 = ok, negative = one `BackendError` variant), the text of the last
 * failure is thread-local, the caller owns every struct it passes, nothing returned is
 * heap-owned by the callee except opaque handles with an explicit destroy call.
 *
 * No torch types appear here: plain pointers, sizes, PODs. There is no CPU fallback:
 * an op/dtype the backend does not implement returns HOLO_ERR_UNSUPPORTED_OP.
 */
#ifndef HOLOGRAM_B200_H
#define HOLOGRAM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: one per BackendError variant (crates/hologram-compute/src/error.rs:6-20) */
#define HOLO_OK 0
#define HOLO_ERR_SLOT_OUT_OF_RANGE (-1) /* BackendError::SlotOutOfRange(slot) */
#define HOLO_ERR_SHAPE_MISMATCH (-2)    /* BackendError::ShapeMismatch{..}   */
#define HOLO_ERR_UNSUPPORTED_OP (-3)    /* BackendError::UnsupportedOp(msg)   */
#define HOLO_ERR_INIT (-4)              /* BackendError::Init(msg)            */
#define HOLO_ERR_DISPATCH (-5)          /* BackendError::Dispatch(msg)        */

/* ---- dtype tags: DTypeId (crates/hologram-types/src/dtype_id.rs:51-74), wire-stable u8 */
#define HOLO_DTYPE_BOOL 0
#define HOLO_DTYPE_U8 1
#define HOLO_DTYPE_I8 2
#define HOLO_DTYPE_U64 3
#define HOLO_DTYPE_I32 4
#define HOLO_DTYPE_I64 5
#define HOLO_DTYPE_F16 6
#define HOLO_DTYPE_BF16 7
#define HOLO_DTYPE_F32 8
#define HOLO_DTYPE_F64 9
#define HOLO_DTYPE_E8CB 11 /* one u8 index of an 8-element codebook block per eight weights; MatMulDequant weight only */
#define HOLO_DTYPE_I4 10 /* two signed nibbles per byte, low nibble first; DequantActivation input only */

/* ---- lut_act ids (crates/hologram-compute/src/kernel_call.rs:877-885) */
#define HOLO_LUT_SIGMOID 0
#define HOLO_LUT_TANH 1
#define HOLO_LUT_GELU 2
#define HOLO_LUT_SILU 3
#define HOLO_LUT_EXP 4
#define HOLO_LUT_ERF 5
#define HOLO_LUT_COUNT 6

/* ---- fused_activation ids (kernel_call.rs:861-870) */
#define HOLO_FUSED_RELU 1
#define HOLO_FUSED_GELU 2
#define HOLO_FUSED_SILU 3
#define HOLO_FUSED_SIGMOID 4
#define HOLO_FUSED_TANH 5
#define HOLO_FUSED_EXP 8

/* ---- KernelCall variant tags. Values are the archive wire discriminants
 * (crates/hologram-archive/src/kernel_codec.rs:19-128) so a decoded .holo call list maps
 * 1:1. Tags >= 0x8000 are extensions with no reference counterpart (documented below). */
#define HOLO_K_NEG 1
#define HOLO_K_ADD 5
#define HOLO_K_SUB 6
#define HOLO_K_MUL 7
#define HOLO_K_RELU 11
#define HOLO_K_SIGMOID 12
#define HOLO_K_TANH 13
#define HOLO_K_GELU 14
#define HOLO_K_SILU 15
#define HOLO_K_EXP 18
#define HOLO_K_SQRT 21
#define HOLO_K_RECIPROCAL 22
#define HOLO_K_CEIL 29
#define HOLO_K_FLOOR 30
#define HOLO_K_ROUND 31
#define HOLO_K_ERF 32
#define HOLO_K_IS_NAN 33
#define HOLO_K_SIGN 34
#define HOLO_K_ABS 35
#define HOLO_K_DIV 36
#define HOLO_K_MOD 38
#define HOLO_K_MIN 39
#define HOLO_K_MAX 40
#define HOLO_K_EQUAL 41
#define HOLO_K_LESS 42
#define HOLO_K_LESS_OR_EQUAL 43
#define HOLO_K_GREATER 44
#define HOLO_K_GREATER_OR_EQUAL 45
#define HOLO_K_MATMUL 46
#define HOLO_K_LAYER_NORM 50
#define HOLO_K_RMS_NORM 51
#define HOLO_K_ADD_RMS_NORM 54
#define HOLO_K_REDUCE_SUM 55
#define HOLO_K_REDUCE_MEAN 56
#define HOLO_K_REDUCE_PROD 57
#define HOLO_K_REDUCE_MIN 58
#define HOLO_K_REDUCE_MAX 59
#define HOLO_K_RESHAPE 60
#define HOLO_K_TRANSPOSE 61
#define HOLO_K_CONCAT 62
#define HOLO_K_SLICE 63
#define HOLO_K_SOFTMAX 64
#define HOLO_K_ATTENTION 69
#define HOLO_K_EXPAND 72
#define HOLO_K_ROTARY 75
#define HOLO_K_WHERE 78
#define HOLO_K_DEQUANTIZE 105
#define HOLO_K_MATMUL_ACTIVATION 106
#define HOLO_K_MATMUL_ADD 107
#define HOLO_K_MATMUL_ADD_ACTIVATION 108 /* kernel_codec.rs D_MMAA: act(A . B + residual), no narrowing between the add and the activation */
#define HOLO_K_MATMUL_DEQUANT_PLAIN 111  /* kernel_codec.rs D_MMDQ: the all-default MatMulDequant ([k,n] weight, f32 activations: "W8A32") */
#define HOLO_K_BROADCAST_BINARY 112
#define HOLO_K_DEQUANT_ACTIVATION 113
#define HOLO_K_GATHER 114
#define HOLO_K_MATMUL_DEQUANT_CODEBOOK 117 /* kernel_codec.rs D_MMDQ3: the same call with a codebook operand bound (E8 codebook weight tier) */
#define HOLO_K_MATMUL_DEQUANT 116 /* the extended wire form (kernel_codec.rs D_MMDQ2); served: output-major W8A8 int8 */
#define HOLO_K_CAST 115
#define HOLO_K_DECODE_ATTENTION 119
#define HOLO_K_KV_CACHE_WRITE 120
#define HOLO_K_DECODE_ATTENTION_VALID 121
/* Extensions (the reference has no KV quantizer op and no quantized-KV attention):
 * QUANTIZE_ROWS_I8 applies the reference's only f32->i8 quantizer, `quantize_row_i8`
 * (crates/hologram-compute/src/cpu/simd.rs:4761-4785), to every row;
 * DECODE_ATTENTION_VALID_Q8 is DecodeAttentionValid over Dequantize'd int8 K/V;
 * ALL_REDUCE is the tensor-parallel sum after o-proj / down-proj. */
#define HOLO_K_QUANTIZE_ROWS_I8 0x8001
#define HOLO_K_DECODE_ATTENTION_VALID_Q8 0x8002
#define HOLO_K_ALL_REDUCE 0x8003
/* RotaryEmbedding followed by QuantizeRowsI8 of its result, one row = one head (fused at load by the
 * session when a RoPE output feeds a row quantizer of the same row length; bit-identical to the pair). */
#define HOLO_K_ROPE_QUANTIZE_ROWS_I8 0x8004

/* BufferRef (crates/hologram-compute/src/workspace.rs:16-24). length == 0 means "the slot's
 * full extent from offset". slot == UINT32_MAX marks an absent optional operand
 * (kernel_call.rs:217-228, 450-458). */
typedef struct HoloBufferRef {
    uint32_t slot;
    uint64_t offset;
    uint64_t length;
} HoloBufferRef;
#define HOLO_NO_SLOT 0xFFFFFFFFu

/* UnaryCall (kernel_call.rs:30-36) */
typedef struct HoloUnaryCall {
    HoloBufferRef input, output;
    uint64_t element_count;
    uint16_t witt_bits;
    uint8_t dtype;
} HoloUnaryCall;

/* BinaryCall (kernel_call.rs:38-46) */
typedef struct HoloBinaryCall {
    HoloBufferRef a, b, output;
    uint64_t element_count;
    uint16_t witt_bits;
    uint8_t dtype;
} HoloBinaryCall;

/* MatMulCall (kernel_call.rs:49-65): A [m,k] row-major, B [k,n] row-major, f32 accumulation */
typedef struct HoloMatMulCall {
    HoloBufferRef a, b, output;
    uint32_t m, k, n;
    uint8_t dtype;
    uint8_t b_packed; /* must be 0: panel packing is f32-only in the reference (compiler.rs:609) */
} HoloMatMulCall;

/* MatMulActivationCall (kernel_call.rs:887-897) */
typedef struct HoloMatMulActivationCall {
    HoloMatMulCall mm;
    uint8_t act; /* HOLO_FUSED_* */
} HoloMatMulActivationCall;

/* MatMulAddCall (kernel_call.rs:899-911) */
typedef struct HoloMatMulAddCall {
    HoloMatMulCall mm;
    HoloBufferRef residual;
} HoloMatMulAddCall;

/* MatMulAddActivationCall (kernel_call.rs:913-929): out = act(A . B + residual). The reference forms it for f32
 * only (session.rs:2220-2226, where no narrowing is skipped); for 16-bit dtypes the product is narrowed once, the sum
 * and the activation are taken in f32 and narrowed once more (cpu/float_kernels.rs:933-936). */
typedef struct HoloMatMulAddActivationCall {
    HoloMatMulCall mm;
    HoloBufferRef residual;
    uint8_t act; /* HOLO_FUSED_* */
} HoloMatMulAddActivationCall;

/* NormCall (kernel_call.rs:423-446); RmsNorm uses x, gamma, output, batch, feature, epsilon_bits */
typedef struct HoloNormCall {
    HoloBufferRef x, gamma, beta, residual, output;
    uint32_t batch, feature, channels, num_groups;
    uint64_t epsilon_bits;
    uint8_t dtype;
} HoloNormCall;

/* MatMulDequantCall (kernel_call.rs:152-213), wire forms 111 / 116 / 117: out = act(A . dequant(Bq) [+ residual]).
 * Served: (1) the output-major W8A8 decode product (bq_omajor = 1, act_quant = 1 = W8A8_TOKEN_SYM): A f32
 * [m,k], Bq i8 / i4 / e8cb [n,k], symmetric per-channel scales f32 [n] (channels = n, inner = 1, zero points all 0),
 * f32 output; every A row quantized with quantize_row_i8, exact i32 dot, one f32 writeback.
 * (2) the [k,n] form with f32 activations (bq_omajor = 0, act_quant = 0, "W8A32", cpu/float_kernels.rs:596-731):
 * Bq i8 / u8 / i4 [k,n], per-tensor (scale_bits, zero_point) or per-channel scales / zero points; every output cell
 * is the reference's ascending-k multiply-add chain over the dequantized weights (for m <= 3 with symmetric
 * per-column i8 scales: the chain over the integer levels, the column scale applied once at the end,
 * cpu/simd.rs:3480-3570). */
typedef struct HoloMatMulDequantCall {
    HoloBufferRef a, bq, scales, zero_points, output;
    uint32_t m, k, n, channels, inner;
    uint8_t quant_dtype, dtype;
    uint32_t scale_bits;
    int32_t zero_point;
    uint8_t bq_omajor, act_quant, act;
    HoloBufferRef residual;
    HoloBufferRef codebook; /* tag 117 only: the model's 256 x 8 i8 codebook (2048 bytes); slot HOLO_NO_SLOT otherwise */
} HoloMatMulDequantCall;

/* SoftmaxCall (kernel_call.rs:549-556): rows of `feature` elements; max, deterministic exp of the
 * shifted row, sum, divide; a row of -inf is all zeros. */
typedef struct HoloSoftmaxCall {
    HoloBufferRef input, output;
    uint32_t batch, feature;
    uint8_t dtype;
} HoloSoftmaxCall;

/* WhereCall (kernel_call.rs:761-769): out[i] = cond[i] != 0 ? a[i] : b[i]; cond is one byte per element. */
typedef struct HoloWhereCall {
    HoloBufferRef cond, a, b, output;
    uint64_t element_count;
    uint8_t dtype;
} HoloWhereCall;

/* DequantActivationCall (kernel_call.rs:265-290): out[i] = act((q[i] - zero_point) as f32 * scale) as f32 for a
 * per-tensor-quantized i8 / u8 / i4 input; act is a HOLO_LUT_* id. The composition is one table over the 256
 * (16) possible codes, built per launch (cpu/kernels.rs:311-381). */
typedef struct HoloDequantActivationCall {
    HoloBufferRef input, output;
    uint64_t element_count;
    uint8_t quant_dtype, act, dtype;
    uint32_t scale_bits;
    int32_t zero_point;
} HoloDequantActivationCall;

/* AttentionCall (kernel_call.rs:575-594): scaled dot-product attention over q [batch, heads, seq, head_dim] and
 * k, v [batch, kv_heads, seq, head_dim] (kv_heads 0 = heads; query head h reads kv head h / (heads / kv_heads));
 * causal: query row i sees keys j <= i; scale_bits: f32 bits of the score multiplier, 0 = 1/sqrt(head_dim). */
typedef struct HoloAttentionCall {
    HoloBufferRef q, k, v, output;
    uint32_t batch, heads, seq, head_dim, kv_heads;
    uint8_t causal;
    uint32_t scale_bits;
    uint8_t dtype;
} HoloAttentionCall;

/* ReduceCall (kernel_call.rs:461-477): fold the axes whose bit is set in axes_mask (0 or rank 0 = all) of a
 * row-major tensor `dims[..rank]`; the output is the keepdims layout (reduced axes collapsed to 1). Every
 * output cell folds its inputs in linear input order, as the CPU loop does; only the full f32 reduction to
 * one cell is order-relaxed there (chunked SIMD), and here. */
typedef struct HoloReduceCall {
    HoloBufferRef input, output;
    uint64_t element_count;
    uint8_t rank;
    uint32_t dims[8];
    uint32_t axes_mask;
    uint8_t keepdims, dtype;
} HoloReduceCall;

/* ExpandCall (kernel_call.rs:539-547): replicate `input` to out_dims; an axis with in_dims[i] == 1 reads
 * index 0, every other axis maps 1:1 (in_dims[i] == out_dims[i]); rank <= 8; any dtype. */
typedef struct HoloExpandCall {
    HoloBufferRef input, output;
    uint8_t rank;
    uint32_t in_dims[8], out_dims[8];
    uint8_t dtype;
} HoloExpandCall;

/* BroadcastBinaryCall (kernel_call.rs:292-317): out[o] = op(small[bcast(o)], other[o]), operands swapped when
 * small_is_lhs == 0; op 0 add, 1 sub, 2 mul; `small` has in_dims (1 on the broadcast axes), `other` and the
 * output have out_dims. */
#define HOLO_BROADCAST_ADD 0
#define HOLO_BROADCAST_SUB 1
#define HOLO_BROADCAST_MUL 2
typedef struct HoloBroadcastBinaryCall {
    HoloBufferRef small, other, output;
    uint8_t rank;
    uint32_t in_dims[8], out_dims[8];
    uint8_t op, small_is_lhs, dtype;
} HoloBroadcastBinaryCall;

/* TransposeCall (kernel_call.rs:491-499): output axis i is input axis perm[i]; rank <= 8 */
typedef struct HoloTransposeCall {
    HoloBufferRef input, output;
    uint8_t rank;
    uint32_t dims[8];
    uint8_t perm[8];
    uint8_t dtype;
} HoloTransposeCall;

/* RoPECall (kernel_call.rs:506-514): cos/sin are full tensors with x's element layout */
typedef struct HoloRoPECall {
    HoloBufferRef x, cos, sin, output;
    uint32_t head_dim;
    uint64_t element_count;
    uint8_t dtype;
} HoloRoPECall;

/* GatherCall (kernel_call.rs:387-403) */
typedef struct HoloGatherCall {
    HoloBufferRef data, indices, output;
    uint64_t outer, axis_dim, inner, num_indices;
    uint8_t idx_dtype, dtype;
} HoloGatherCall;

/* CastCall (kernel_call.rs:411-419) */
typedef struct HoloCastCall {
    HoloBufferRef input, output;
    uint64_t element_count;
    uint8_t src_dtype, dst_dtype;
} HoloCastCall;

/* LayoutCall (kernel_call.rs:479-485): Reshape is a byte copy when dispatched */
typedef struct HoloLayoutCall {
    HoloBufferRef input, output;
    uint64_t element_count;
    uint8_t dtype;
} HoloLayoutCall;

/* DequantizeCall (kernel_call.rs:782-818); i8/u8 sources, per-tensor or per-channel */
typedef struct HoloDequantizeCall {
    HoloBufferRef input, scales, zero_points, output;
    uint64_t element_count;
    uint32_t channels, inner;
    uint8_t quant_dtype, dtype;
    uint32_t scale_bits;
    int32_t zero_point;
} HoloDequantizeCall;

/* KvCacheWriteCall (kernel_call.rs:742-759). When cache and output resolve to the same
 * device range the write is the O(new_rows) in-place move the executor performs
 * (crates/hologram-exec/src/session.rs:1313-1370); otherwise the honest O(bucket) copy. */
typedef struct HoloKvCacheWriteCall {
    HoloBufferRef cache, new_rows_buf, pos, output;
    uint32_t planes, bucket_rows, new_rows, row_bytes;
} HoloKvCacheWriteCall;

/* DecodeAttentionCall (kernel_call.rs:632-655), the additive-mask form: every past and new key
 * takes part, `mask` is f32 [q_rows, past_len + new_len] shared by batch and heads and is added to
 * the scaled score (-inf erases a key exactly); a row whose keys are all erased is the zero
 * vector. q_rows is independent of new_len; past_len + new_len must be at least 1. */
typedef struct HoloDecodeAttentionCall {
    HoloBufferRef q, k_past, v_past, k_new, v_new, mask, output;
    uint32_t batch, heads, kv_heads, q_rows, past_len, new_len, head_dim, scale_bits;
    uint8_t dtype;
} HoloDecodeAttentionCall;

/* DecodeAttentionValidCall (kernel_call.rs:691-716) */
typedef struct HoloDecodeAttentionValidCall {
    HoloBufferRef q, k_past, v_past, k_new, v_new, valid_len, output;
    uint32_t batch, heads, kv_heads, q_rows, past_len, new_len, head_dim, scale_bits;
    uint8_t dtype;
} HoloDecodeAttentionValidCall;

/* Extension. Rows of `row_len` values of `dtype` (f32/bf16/f16) -> i8 codes [rows,row_len]
 * and f32 scales [rows], bit-for-bit `quantize_row_i8` (simd.rs:4761-4785); an all-zero row
 * gives zero codes and scale 0.0. */
typedef struct HoloQuantizeRowsI8Call {
    HoloBufferRef input, codes, scales;
    uint64_t rows;
    uint32_t row_len;
    uint8_t dtype;
} HoloQuantizeRowsI8Call;

/* Extension. DecodeAttentionValid whose K/V operands are int8 codes [b,kv,rows,d] with f32
 * per-row scales [b,kv,rows]; q and output have `dtype`. Defined as the reference
 * composition Cast(q) / Dequantize(K,V per row, zero-point 0) / DecodeAttentionValid(f32) /
 * Cast(output). */
typedef struct HoloDecodeAttentionValidQ8Call {
    HoloBufferRef q, k_past, k_past_scales, v_past, v_past_scales;
    HoloBufferRef k_new, k_new_scales, v_new, v_new_scales, valid_len, output;
    uint32_t batch, heads, kv_heads, q_rows, past_len, new_len, head_dim, scale_bits;
    uint8_t dtype;
} HoloDecodeAttentionValidQ8Call;

/* Extension: rope_output = RoPE(x, cos, sin) (RoPECall semantics, head_dim = the row length), then
 * codes / scales = QuantizeRowsI8(rope_output). */
typedef struct HoloRopeQuantizeCall {
    HoloBufferRef x, cos, sin, rope_output, codes, scales;
    uint64_t rows;
    uint32_t row_len;
    uint8_t dtype;
} HoloRopeQuantizeCall;

/* Extension. In-place sum over the context's tensor-parallel group (NCCL); a no-op when the
 * context has no group. */
typedef struct HoloAllReduceCall {
    HoloBufferRef buffer;
    uint64_t element_count;
    uint8_t dtype;
} HoloAllReduceCall;

/* The tagged union standing in for `enum KernelCall` (kernel_call.rs:1146-1276). */
typedef struct HoloKernelCall {
    uint16_t kind; /* HOLO_K_* */
    union {
        HoloUnaryCall unary;            /* SIGMOID TANH GELU SILU EXP ERF */
        HoloBinaryCall binary;          /* ADD MUL CONCAT (out = a || b, extents taken from the BufferRefs) */
        HoloMatMulCall matmul;          /* MATMUL */
        HoloMatMulActivationCall matmul_activation;
        HoloMatMulAddCall matmul_add;
        HoloMatMulAddActivationCall matmul_add_activation;
        HoloMatMulDequantCall matmul_dequant;
        HoloNormCall norm;              /* RMS_NORM, ADD_RMS_NORM (norm of x + residual) */
        HoloRoPECall rope;              /* ROTARY */
        HoloGatherCall gather;
        HoloCastCall cast;
        HoloLayoutCall layout;          /* RESHAPE SLICE (contiguous copies; a slice's start is the input ref's offset) */
        HoloTransposeCall transpose;
        HoloSoftmaxCall softmax;
        HoloExpandCall expand;
        HoloReduceCall reduce;
        HoloAttentionCall attention;
        HoloDequantActivationCall dequant_activation;
        HoloWhereCall where;
        HoloBroadcastBinaryCall broadcast_binary;
        HoloDequantizeCall dequantize;
        HoloKvCacheWriteCall kv_cache_write;
        HoloDecodeAttentionCall decode_attention;
        HoloDecodeAttentionValidCall decode_attention_valid;
        HoloQuantizeRowsI8Call quantize_rows_i8;
        HoloDecodeAttentionValidQ8Call decode_attention_valid_q8;
        HoloAllReduceCall all_reduce;
        HoloRopeQuantizeCall rope_quantize;
    } u;
} HoloKernelCall;

typedef struct holo_b200_ctx holo_b200_ctx;             /* per-GPU backend state (the `Backend` impl) */
typedef struct holo_b200_workspace holo_b200_workspace; /* device-resident `Workspace` */

/* ---- errors (hologram-ffi src/lib.rs:48-92 convention) */
/* Text of the calling thread's last failure ("" if none). Valid until the next failing call
 * on this thread. */
const char* holo_b200_last_error(void);
/* The slot number attached to the last HOLO_ERR_SLOT_OUT_OF_RANGE on this thread. */
uint32_t holo_b200_last_error_slot(void);

/* ---- context: replaces `CpuBackend::new()` (crates/hologram-compute/src/cpu.rs:60-86).
 * Creates a stream on `device`, uploads nothing yet; LUT tables are built on device on first
 * use of each (activation, dtype) pair, as cpu/lut.rs:38-72 does lazily on the host. */
int32_t holo_b200_ctx_create(int32_t device, holo_b200_ctx** out);
void holo_b200_ctx_destroy(holo_b200_ctx* ctx);
/* The CUDA stream (cudaStream_t) every dispatch is ordered on. */
void* holo_b200_ctx_stream(holo_b200_ctx* ctx);
/* Order every later dispatch on a caller-owned stream instead (e.g. the host framework's
 * current stream, so its events bracket these kernels). */
int32_t holo_b200_ctx_set_stream(holo_b200_ctx* ctx, void* cuda_stream);
/* Wait for the stream; also reports device-side failures recorded since the last check
 * (an out-of-range Gather index, a bounded wait that gave up). */
int32_t holo_b200_ctx_synchronize(holo_b200_ctx* ctx);
/* Number of this library's kernels launched through the context since creation. */
uint64_t holo_b200_ctx_launch_count(holo_b200_ctx* ctx);
/* Install a 65536-entry table for (lut_act, dtype) instead of the built-in one (tables are
 * data: a table generated by the reference itself can be dropped in unchanged). */
int32_t holo_b200_ctx_set_lut_table(holo_b200_ctx* ctx, uint8_t lut_act, uint8_t dtype, const uint16_t* table65536);
/* Copy the table in use for (lut_act, dtype) to the host. */
int32_t holo_b200_ctx_get_lut_table(holo_b200_ctx* ctx, uint8_t lut_act, uint8_t dtype, uint16_t* table65536);

/* ---- device workspace: replaces the `Workspace` trait object the executor passes
 * (workspace.rs:26-55; implemented by BufferArena, crates/hologram-exec/src/buffer.rs:955-999).
 * A table of `n_slots` slots, each bound to a device range. */
int32_t holo_b200_workspace_create(holo_b200_ctx* ctx, uint32_t n_slots, holo_b200_workspace** out);
void holo_b200_workspace_destroy(holo_b200_workspace* ws);
/* Allocate (or re-allocate) an owned, zero-filled device buffer of `bytes` for `slot`
 * (bind_fresh, buffer.rs:427; zero-on-reuse, buffer.rs:86-108). 256-byte aligned. */
int32_t holo_b200_workspace_alloc(holo_b200_workspace* ws, uint32_t slot, uint64_t bytes);
/* Bind `slot` to caller-owned device memory (bind_resident / bind_view, buffer.rs:437;
 * a memo hit is this pointer rebind, no host round-trip). */
int32_t holo_b200_workspace_bind(holo_b200_workspace* ws, uint32_t slot, void* device_ptr, uint64_t bytes);
/* Device pointer and extent of a slot. */
int32_t holo_b200_workspace_slot(holo_b200_workspace* ws, uint32_t slot, void** device_ptr, uint64_t* bytes);
/* Host <-> device copies of a slot range (Workspace::write / ::read at graph boundaries;
 * resolve, buffer.rs:887). Ordered on the context stream; download synchronises. */
int32_t holo_b200_workspace_upload(holo_b200_workspace* ws, HoloBufferRef dst, const void* host, uint64_t bytes);
int32_t holo_b200_workspace_download(holo_b200_workspace* ws, HoloBufferRef src, void* host, uint64_t bytes);

/* ---- dispatch: replaces `Backend::dispatch` (backend.rs:12-14; CPU body cpu/kernels.rs:16-181).
 * Validates geometry and slot extents first (fail loud, nothing written on error), then
 * enqueues the kernel(s) on the context stream and returns without synchronising. */
int32_t holo_b200_dispatch(holo_b200_ctx* ctx, const HoloKernelCall* call, holo_b200_workspace* ws);

/* Host-memory workspace form: the call's BufferRefs index `host_slots` (pointer + byte size
 * per slot, the reference tests' `TestWorkspace { slots: Vec<Vec<u8>> }`, tests/lut.rs:13-49).
 * Operands are staged to the device, the call dispatched, the output range copied back, and
 * the call returns after synchronising — the per-call upload/dispatch/readback shape of the
 * reference's own GPU backends (wgpu_backend/mod.rs:157-268). Host buffers should be pinned
 * for full transfer speed but need not be. */
typedef struct HoloHostSlot {
    void* ptr;
    uint64_t bytes;
} HoloHostSlot;
int32_t holo_b200_dispatch_host(holo_b200_ctx* ctx, const HoloKernelCall* call, HoloHostSlot* host_slots,
                                uint32_t n_slots);

/* ---- archive session: the device-side counterpart of `InferenceSession::load` / `execute`
 * (crates/hologram-exec/src/session.rs:399-792, 846-932) for archives made of the served call
 * variants. Load parses the `.holo` image (BLAKE3 footer and weight fingerprints checked when
 * `verify` != 0), applies the load-time MatMul epilogue fusion (session.rs:2150-2377), places
 * every slot in HBM, uploads constants once, and realises input-port -> output-port
 * KvCacheWrite calls as in-place moves (session.rs:1313-1370). The image may be freed after
 * load returns. */
typedef struct holo_b200_session holo_b200_session;
int32_t holo_b200_session_load(holo_b200_ctx* ctx, const uint8_t* archive, uint64_t len, int32_t verify,
                               holo_b200_session** out);
void holo_b200_session_destroy(holo_b200_session* s);
/* The session's device workspace (owned by the session): upload inputs / download outputs
 * through it, or bind caller-owned device memory to a port's slot. */
holo_b200_workspace* holo_b200_session_workspace(holo_b200_session* s);
/* Counters (session.rs:1294-1303, 1385-1440 style): calls after fusion, fused pairs, in-place
 * KV moves, port counts, bytes of HBM held by slots. Any pointer may be NULL. */
int32_t holo_b200_session_info(holo_b200_session* s, uint32_t* n_calls, uint32_t* n_fused, uint32_t* n_moved,
                               uint32_t* n_inputs, uint32_t* n_outputs, uint64_t* device_bytes);
/* What one walk launches: the number of launch nodes, and how many calls were absorbed into
 * merged sibling matmuls (consecutive MatMul / MatMulActivation calls over the same A and
 * constant weights run as one product against column-concatenated weights, each call keeping
 * its own output buffer and epilogue). */
int32_t holo_b200_session_nodes(holo_b200_session* s, uint32_t* n_nodes, uint32_t* n_merged_calls);
/* Port `index` of the Inputs (is_output == 0) or Outputs section (writer.rs:246-263). */
int32_t holo_b200_session_port(holo_b200_session* s, int32_t is_output, uint32_t index, char* name, uint32_t name_cap,
                               uint32_t* slot, uint64_t* element_count, uint8_t* dtype);
/* Copy of call `index` in post-fusion execution order. */
int32_t holo_b200_session_call(holo_b200_session* s, uint32_t index, HoloKernelCall* out);
/* One walk over the call list (compute_and_label, session.rs:1052-1289, without the κ
 * bookkeeping): every call is enqueued on the context stream; returns without synchronising. */
int32_t holo_b200_session_execute(holo_b200_session* s);
/* Capture one walk into a CUDA graph that later `execute` calls replay. Call after at least
 * one plain execute. */
int32_t holo_b200_session_capture(holo_b200_session* s);

/* Parse an archive image on the host only (header, section table, call codec, ports,
 * constants; BLAKE3 footer and weight fingerprints when `verify` != 0): the HoloLoader checks
 * (crates/hologram-archive/src/loader.rs:141-267). Needs no device. */
int32_t holo_b200_archive_check(const uint8_t* archive, uint64_t len, int32_t verify, uint32_t* n_calls,
                                uint32_t* n_inputs, uint32_t* n_outputs, uint32_t* n_constants);

/* Decode attention over an int8 KV cache for callers that must not allocate device memory.
 * It has no counterpart in the reference; it is DecodeAttentionValidQ8 (q_rows = new_len = 1)
 * taken with plain device pointers and a CUDA stream instead of a context and a workspace.
 * The split-KV partial results go to a 16 MiB array built into the library (each GPU that loads
 * the library keeps that array until the process exits) rather than to the context's growable
 * scratch buffer, so the call performs no cudaMalloc / cudaFree and needs no context.
 * Limits: head_dim 128; heads / kv_heads <= 4; past_len a multiple of 4 and >= 4; code and scale
 * pointers 16-byte aligned; shapes whose partials exceed the array ((2 * SM count + 2 * batch *
 * kv_heads) * 4 * 130 floats: about 3800 (batch, kv head) planes) are refused with
 * HOLO_ERR_UNSUPPORTED_OP.
 * The first call on each device looks the array up (the device of the calling thread must be the
 * stream's device); make that first call before any stream capture begins. All calls share the
 * array: two calls that overlap on the GPU (different streams) race on it. Enqueues on
 * `cuda_stream` and returns without synchronising; a failure inside the kernel (a bounded wait
 * that gave up: nothing is written to `out`) is reported by the status call below, and until it
 * has been reported the kernels of later calls return at once without writing. */
int32_t holo_b200_decode_attention_q8_static(void* cuda_stream, const void* q, const int8_t* k_past,
                                             const float* k_past_scales, const int8_t* v_past, const float* v_past_scales,
                                             const int8_t* k_new, const float* k_new_scales, const int8_t* v_new,
                                             const float* v_new_scales, const uint32_t* valid_len, void* out,
                                             uint32_t batch, uint32_t heads, uint32_t kv_heads, uint32_t past_len,
                                             uint32_t head_dim, uint32_t scale_bits, uint8_t dtype);
/* Companion of the entry point above (no counterpart in the reference either): waits for
 * `cuda_stream`, reads the 4-byte status word of the built-in array back (no allocation) and
 * returns HOLO_ERR_DISPATCH if a bounded device-side wait gave up since the last query, clearing
 * the record; HOLO_OK otherwise. Call it where the caller synchronises anyway (per step). */
int32_t holo_b200_decode_attention_q8_static_status(void* cuda_stream);

/* ---- content-addressed execution (crates/hologram-exec/src/session.rs:942-984 execute_addressed,
 * :1052-1289 the walk; labels crates/hologram-archive/src/address.rs:83-116, :197-221).
 * A label is 71 ASCII bytes, "blake3:" + 64 hex digits. Load the session with HOLO_SESSION_ADDRESSED
 * or-ed into `verify`. Values live in a label-keyed pool of device buffers (the device-resident
 * BufferArena, crates/hologram-exec/src/buffer.rs:149-207): intern the inputs (or feed a previous
 * call's output labels straight back in), pass their labels in port order and receive the outputs'
 * labels. A node whose derived label is already resident is bound by pointer and not dispatched; a
 * repeat of the same input labels is answered from the memo without touching the device; a
 * KvCacheWrite whose cache value is uniquely owned is realised as the in-place move (session.rs:1313-1370).
 * Interior values carry the cheap derivation (derive_label); a graph output is retained, and reported,
 * under the boundary form (derive_label_boundary, address.rs:197-221). An output that has no derivable
 * label (it depends on a value the labels do not see, e.g. a tensor-parallel sum) is labelled by its bytes
 * (the only place a result is read back and hashed).
 * Every input label must be resident (interned since the last walk, returned by the last walk, leased or
 * pinned); otherwise the call is refused before any state changes (session.rs:959-971). */
#define HOLO_SESSION_VERIFY 1
#define HOLO_SESSION_ADDRESSED 2
/* The operand list the reference derives a norm's label from is x, gamma, beta (kernel_call.rs:1612-1616),
 * so AddRmsNorm(x, r1) and AddRmsNorm(x, r2) share a label there. That is the default here too (labels are
 * byte-identical to the reference's). With this flag the residual operand is appended, so that two sums
 * over different residuals never share a label. */
#define HOLO_SESSION_LABEL_RESIDUAL 4
typedef struct HoloAddressedStats {
    uint32_t dispatched; /* calls launched by this walk */
    uint32_t skipped;    /* calls answered by a resident value (moves included, as in the reference's last_skipped) */
    uint32_t memo_hit;   /* 1: the whole graph was answered from the memo */
    uint64_t pool_bytes; /* device bytes the label pool has allocated (released buffers included) */
    uint32_t moved;      /* KvCacheWrite calls realised as the in-place move */
    uint32_t paged_in;   /* weights paged in from the provider so far (load_paged sessions) */
} HoloAddressedStats;
int32_t holo_b200_session_execute_addressed(holo_b200_session* s, const uint8_t* input_labels, uint32_t n_inputs,
                                            uint8_t* output_labels, uint32_t n_outputs, HoloAddressedStats* stats);
/* intern_input (session.rs:1018-1022): hash `len` host bytes once, store them in the pool under that
 * label (no slot is bound) and return the label; use it as an input of execute_addressed. */
int32_t holo_b200_session_intern_input(holo_b200_session* s, const void* host, uint64_t len, uint8_t out71[71]);
/* resolve (session.rs:1027-1029): copy the bytes of a resident label to the host (at most `cap`
 * bytes; *len receives the value's length). *resident = 0 when the label is not in the pool. Synchronises. */
int32_t holo_b200_session_resolve(holo_b200_session* s, const uint8_t label71[71], void* host, uint64_t cap, uint64_t* len,
                                  int32_t* resident);
/* retain_label / release_label (session.rs:1000-1012; buffer.rs:795-836): a leased value survives every
 * walk until released (residency by ownership, not recency) and refuses the in-place KvCacheWrite move, so
 * a step on a leased cache takes the honest copy and the leased pre-image stays bit-intact: the rollback
 * primitive of speculative decoding and branch search. Refcounted. *ok = 0 when the label is not resident
 * (retain) or holds no lease (release). */
int32_t holo_b200_session_retain_label(holo_b200_session* s, const uint8_t label71[71], int32_t* ok);
int32_t holo_b200_session_release_label(holo_b200_session* s, const uint8_t label71[71], int32_t* ok);
/* leased_count (session.rs:1479). */
uint32_t holo_b200_session_leased_count(holo_b200_session* s);
/* address_bytes: the label of a leaf value (address.rs:83-86). */
int32_t holo_b200_label_bytes(const uint8_t* data, uint64_t len, uint8_t out71[71]);
/* derive_label: BLAKE3(opcode LE16 || params || labels...) as a label (address.rs:108-116). */
int32_t holo_b200_label_derive(uint16_t opcode, const uint8_t* params, uint32_t params_len, const uint8_t* labels,
                               uint32_t n_labels, uint8_t out71[71]);
/* derive_label_boundary (address.rs:197-221): the label of (opcode LE16 || params), then every operand label
 * folded in order through the ordered product address_bytes(left digest || right digest)
 * (crates/hologram-archive/src/compose.rs:154-164); with no operand the op label is composed with itself. */
int32_t holo_b200_label_derive_boundary(uint16_t opcode, const uint8_t* params, uint32_t params_len, const uint8_t* labels,
                                        uint32_t n_labels, uint8_t out71[71]);
/* KernelCall::op_signature (kernel_call.rs:1321-1516): opcode and scalar parameter bytes. */
int32_t holo_b200_op_signature(const HoloKernelCall* call, uint16_t* opcode, uint8_t params64[64], uint32_t* params_len);

/* ---- paged weights (session.rs:417 load_paged; buffer.rs:491 pin_lazy, :650 page_and_bind_group).
 * The session keeps a bounded window of HBM over a host-side weight set instead of a full copy:
 * constants stored by reference (the large bodies) are declared by fingerprint at load, paged in from
 * the provider (ideally pinned host memory) right before the first call that reads them, and evicted
 * least-recently-used to keep the resident bytes within `budget_bytes` (0 = never evict). A model that
 * fits the budget pages each weight once and then runs like a fully resident load; results are
 * bit-identical either way. The archive may omit the Weights section (a weightless archive).
 * Implies HOLO_SESSION_ADDRESSED. The provider must outlive the session. */
typedef struct HoloWeightProvider {
    void* user;
    /* full body length for a fingerprint, or -1 if the provider does not have it (weight.rs:56) */
    int64_t (*size)(void* user, const uint8_t fingerprint[32]);
    /* pointer to bytes [offset, offset + len) of the body, valid until the session is destroyed, or NULL (weight.rs:61) */
    const void* (*get_range)(void* user, const uint8_t fingerprint[32], uint64_t offset, uint64_t len);
} HoloWeightProvider;
int32_t holo_b200_session_load_paged(holo_b200_ctx* ctx, const uint8_t* archive, uint64_t len, int32_t verify,
                                     const HoloWeightProvider* provider, uint64_t budget_bytes, holo_b200_session** out);

/* ---- memory-tier report (crates/hologram-exec/src/coherence.rs:78-154, session.rs:797 tier_report;
 * crates/hologram-types/src/memory_tier.rs:41-51). Every call has a tier that is a pure function of its
 * dtype's bit width (<= 8: CpuL1, <= 16: CpuL2, <= 24: CpuMain, else Device; layout-only calls CpuMain);
 * a policy maps it to the effective tier and the level-boundary migration schedule follows from it.
 * This backend runs every call on the device whatever its tier: HOLO_TIER_FORCE_ALL_DEVICE is the policy
 * it executes under (no slot ever migrates after its first upload); the other policies are reported
 * for comparison with the reference's planner, nothing is executed differently. */
#define HOLO_TIER_COMPILED 0
#define HOLO_TIER_FORCE_ALL_CPU 1
#define HOLO_TIER_FORCE_ALL_DEVICE 2
typedef struct HoloTierReport {
    uint32_t cpu_l1_calls, cpu_l2_calls, cpu_main_calls, device_calls;
    uint32_t total_migration_slots, levels_with_migrations;
} HoloTierReport;
int32_t holo_b200_session_tier_report(holo_b200_session* s, int32_t policy, HoloTierReport* out);

/* ---- label-keyed buffer pool on its own (the BufferArena operations the executor calls,
 * buffer.rs:273-952). `ctx` NULL gives a pool over plain host memory: the same table logic with no
 * device, for unit tests of the residency rules. Labels are 71 bytes. Functions returning int32_t
 * report 1 / 0 for the reference's bool results and a negative status on failure. */
typedef struct holo_b200_pool holo_b200_pool;
int32_t holo_b200_pool_create(holo_b200_ctx* ctx, holo_b200_pool** out);
void holo_b200_pool_destroy(holo_b200_pool* p);
int32_t holo_b200_pool_rebind_reset(holo_b200_pool* p, uint32_t n_slots);
int32_t holo_b200_pool_store_unbound(holo_b200_pool* p, const uint8_t label71[71], const void* host, uint64_t len);
int32_t holo_b200_pool_pin_bytes(holo_b200_pool* p, const uint8_t label71[71], const void* host, uint64_t len);
int32_t holo_b200_pool_bind_fresh(holo_b200_pool* p, uint32_t slot, uint64_t len);
int32_t holo_b200_pool_bind_resident(holo_b200_pool* p, uint32_t slot, const uint8_t label71[71]);
int32_t holo_b200_pool_retain(holo_b200_pool* p, uint32_t slot, const uint8_t label71[71]);
/* steal_transient + bind_stolen: on success (1) the label is retired and its buffer is bound to `out_slot` */
int32_t holo_b200_pool_steal_transient(holo_b200_pool* p, const uint8_t label71[71], const uint32_t* allowed_slots,
                                       uint32_t n_allowed, uint32_t out_slot);
int32_t holo_b200_pool_lease(holo_b200_pool* p, const uint8_t label71[71]);
int32_t holo_b200_pool_release(holo_b200_pool* p, const uint8_t label71[71]);
int32_t holo_b200_pool_resident(holo_b200_pool* p, const uint8_t label71[71]);
int32_t holo_b200_pool_bindable_input(holo_b200_pool* p, const uint8_t label71[71]);
int32_t holo_b200_pool_resolve(holo_b200_pool* p, const uint8_t label71[71], void* host, uint64_t cap, uint64_t* len);
/* pointer and length of the buffer bound to a slot (1), or 0 when the slot is unbound */
int32_t holo_b200_pool_slot(holo_b200_pool* p, uint32_t slot, void** ptr, uint64_t* len);
/* write host bytes into the buffer bound to a slot (the role a kernel's output plays) */
int32_t holo_b200_pool_write_slot(holo_b200_pool* p, uint32_t slot, const void* host, uint64_t len);
int32_t holo_b200_pool_set_lazy_budget(holo_b200_pool* p, uint64_t bytes);
int32_t holo_b200_pool_pin_lazy(holo_b200_pool* p, const uint8_t label71[71], const uint8_t fingerprint[32], uint64_t size);
int32_t holo_b200_pool_page_and_bind(holo_b200_pool* p, const uint32_t* slots, const uint8_t* labels, uint32_t n,
                                     const HoloWeightProvider* provider);
typedef struct HoloPoolStats {
    uint64_t owned_bytes, lazy_resident_bytes, pages_in;
    uint32_t leased, transient, released;
} HoloPoolStats;
int32_t holo_b200_pool_stats(holo_b200_pool* p, HoloPoolStats* out);

/* ---- tensor-parallel group (no reference counterpart: the reference is single-device).
 * `nccl_unique_id` is the 128-byte ncclUniqueId produced by holo_b200_nccl_unique_id on rank 0
 * and broadcast by the host launcher. */
int32_t holo_b200_nccl_unique_id(uint8_t out128[128]);
int32_t holo_b200_ctx_init_tp(holo_b200_ctx* ctx, const uint8_t nccl_unique_id[128], int32_t rank, int32_t world);
/* The same with a host-side time limit on the group's set-up: the communicator is created in NCCL's
 * non-blocking mode and polled (ncclCommGetAsyncError); if the group has not formed after `timeout_ms`
 * (a rank that never joins, a wrong world size on one rank) the attempt is aborted on the host and
 * HOLO_ERR_INIT is returned. Nothing is enqueued on the GPU before the group has formed. 0 = no limit.
 * holo_b200_ctx_init_tp uses HOLO_TP_INIT_TIMEOUT_MS (default 120000). */
int32_t holo_b200_ctx_init_tp_timeout(holo_b200_ctx* ctx, const uint8_t nccl_unique_id[128], int32_t rank, int32_t world,
                                      uint32_t timeout_ms);
/* How the group's all-reduces of decode-sized 16-bit messages travel: 0 = no group, 1 = NCCL,
 * 2 = the library's own one-shot kernel over peer memory (CUDA IPC mailboxes; every rank sums
 * in rank order, so all ranks hold identical bits). Set HOLO_TP_P2P=0 to stay on NCCL. */
int32_t holo_b200_ctx_tp_transport(holo_b200_ctx* ctx);
/* Self-check of the peer-memory all-reduce on ONE GPU: `world` (2..8) ranks run as one cooperative
 * launch of the same device code, every mailbox in local memory. partials / residuals / outs are
 * host arrays of `world` device pointers to `count` 16-bit elements each (residuals or its entries
 * may be null; outs may alias partials). Synchronises. */
int32_t holo_b200_tp_emulate_all_reduce(holo_b200_ctx* ctx, int32_t world, const void* const* partials, const void* const* residuals,
                                        void* const* outs, uint64_t count, uint8_t dtype, int32_t repeats);
/* The same self-check with a peer that never sends: the CTAs of `withheld_rank` (-1 = none) return at once,
 * so the other ranks' polls of its units run out after `poll_limit` polls (0 = the library's limit), every
 * waiting thread gives up, the kernel ends and the call returns HOLO_ERR_DISPATCH (the context stays
 * usable: the next call works). This is how a dead peer surfaces on the host. */
int32_t holo_b200_tp_emulate_all_reduce_ex(holo_b200_ctx* ctx, int32_t world, const void* const* partials, const void* const* residuals,
                                           void* const* outs, uint64_t count, uint8_t dtype, int32_t repeats, int32_t withheld_rank,
                                           uint32_t poll_limit);

/* Library version / build info string (static storage). */
const char* holo_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HOLOGRAM_B200_H */
