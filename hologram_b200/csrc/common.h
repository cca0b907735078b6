// Internal declarations shared by the backend's translation units. Not part of the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/hologram_b200.h"

struct HoloSlot {
    void* ptr = nullptr;
    uint64_t bytes = 0;
    bool owned = false;
    // a session's weight that none of its calls writes (set at load, cleared by a rebind): kernels may read it
    // without waiting for the launch before them
    bool constant = false;
};

// One small op of a batched launch (see micro_batch_kernel).
enum { HOLO_MICRO_KV_WRITE = 0, HOLO_MICRO_ROPE, HOLO_MICRO_QUANT_VEC, HOLO_MICRO_QUANT, HOLO_MICRO_BINARY_VEC, HOLO_MICRO_BINARY, HOLO_MICRO_ROPE_QUANT };
struct HoloMicroOp {
    uint32_t kind, cta_begin, cta_count, dtype;
    const void *p0, *p1, *p2;
    void *o0, *o1, *o2;
    uint64_t n;
    uint32_t a, b, c, d;
};

struct holo_b200_ctx {
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    uint64_t launches = 0;
    uint16_t* lut[HOLO_LUT_COUNT][2] = {};  // device tables, [act][0 = f16, 1 = bf16]
    // split-KV partials of the decode attention / split-K partials of the skinny GEMM
    void* scratch = nullptr;
    uint64_t scratch_bytes = 0;
    // device staging arena used by the host-workspace dispatch form
    void* stage = nullptr;
    uint64_t stage_bytes = 0;
    // device-side error word (bounded waits record where they gave up)
    uint32_t* dev_status = nullptr;
    uint32_t* attn_arrivals = nullptr;  // 65536 counters, zero between launches (decode attention)
    // launch every kernel with programmatic stream serialization (HOLO_PDL=0 turns it off)
    bool pdl = true;
    // set by a session while it records a batch: launchers append here instead of launching
    std::vector<HoloMicroOp>* record = nullptr;
    bool record_failed = false;
    // tensor-parallel group
    void* nccl_comm = nullptr;
    bool nccl_nonblocking = false;   // the communicator was made in NCCL's non-blocking mode: calls on it are polled to completion
    int tp_rank = 0, tp_world = 1;
    // peer-memory transport: every rank's mailbox as mapped here, per-chunk epoch counters
    bool tp_p2p = false;
    uint8_t* tp_mailbox[8] = {};
    uint32_t* tp_epochs = nullptr;
};

struct holo_b200_workspace {
    holo_b200_ctx* ctx = nullptr;
    std::vector<HoloSlot> slots;
};

// ---- errors -------------------------------------------------------------------------------
int32_t holo_fail(int32_t code, const char* fmt, ...);
int32_t holo_fail_slot(uint32_t slot, const char* what);
int32_t holo_cuda_fail(cudaError_t e, const char* where);
#define HOLO_CUDA(expr)                                             \
    do {                                                            \
        cudaError_t _e = (expr);                                    \
        if (_e != cudaSuccess) return holo_cuda_fail(_e, #expr);    \
    } while (0)
#define HOLO_TRY(expr)                 \
    do {                               \
        int32_t _rc = (expr);          \
        if (_rc != HOLO_OK) return _rc; \
    } while (0)

// Resolve a BufferRef to a device range holding at least `need` bytes
// (length == 0 => the slot's extent from offset; workspace.rs:21-23, buffer.rs:318-327).
int32_t holo_resolve(holo_b200_workspace* ws, HoloBufferRef ref, uint64_t need, uint8_t** ptr, uint64_t* extent);
// Grow the context scratch buffer to at least `bytes` (never shrinks).
int32_t holo_ensure_scratch(holo_b200_ctx* ctx, uint64_t bytes);
static inline size_t holo_dtype_size(uint8_t dtype) {
    switch (dtype) {
        case HOLO_DTYPE_BOOL: case HOLO_DTYPE_U8: case HOLO_DTYPE_I8: return 1;
        case HOLO_DTYPE_F16: case HOLO_DTYPE_BF16: return 2;
        case HOLO_DTYPE_I32: case HOLO_DTYPE_F32: return 4;
        case HOLO_DTYPE_U64: case HOLO_DTYPE_I64: case HOLO_DTYPE_F64: return 8;
        default: return 0;
    }
}
static inline bool holo_is_compute_float(uint8_t d) {
    return d == HOLO_DTYPE_F16 || d == HOLO_DTYPE_BF16 || d == HOLO_DTYPE_F32;
}

// Every BufferRef of a call; `out_bytes` > 0 marks a written operand and gives the number of
// bytes the kernel produces there (inputs carry 0).
struct HoloRefList {
    HoloBufferRef* refs[12];
    uint64_t out_bytes[12];
    bool written[12];
    int n = 0;
    void in(HoloBufferRef* r) {
        refs[n] = r;
        out_bytes[n] = 0;
        written[n] = false;
        ++n;
    }
    void out(HoloBufferRef* r, uint64_t bytes) {
        refs[n] = r;
        out_bytes[n] = bytes;
        written[n] = true;
        ++n;
    }
};
bool holo_collect_refs(HoloKernelCall* c, HoloRefList* l);
// Backend::dispatch body shared by the C entry points and the session walk.
int32_t holo_dispatch_internal(holo_b200_ctx* ctx, const HoloKernelCall* call, holo_b200_workspace* ws);

#ifdef __CUDACC__
// Programmatic dependent launch. Every kernel of the library starts with holo_pdl_trigger()
// ("my successor may be scheduled") and calls holo_pdl_wait() before its first access to global
// memory ("my predecessor has finished and its writes are visible"). Launched through
// holo_launch_kernel with the context's pdl flag set, a kernel's CTAs are then placed on SMs,
// and run their prologue (barrier set-up, TMEM allocation), while the previous kernel drains,
// instead of after it has fully retired; without the attribute both instructions do nothing.
// Because every kernel waits before it reads or writes global memory, and completion of a
// kernel implies completion of everything it waited for, ordering along the stream is kept.
__device__ __forceinline__ void holo_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void holo_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// A thread-block cluster of `cluster` CTAs along grid x (cluster_x) or grid z (cluster_z); 1 = no cluster.
template <typename... KArgs, typename... Args>
static inline cudaError_t holo_launch_kernel_cluster(holo_b200_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                                     unsigned cluster_x, unsigned cluster_z, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    unsigned na = 0;
    if (ctx->pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (cluster_z > 1 || cluster_x > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = cluster_x > 1 ? cluster_x : 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = cluster_z > 1 ? cluster_z : 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// cluster_z > 1 makes grid z a thread-block cluster dimension.
template <typename... KArgs, typename... Args>
static inline cudaError_t holo_launch_kernel(holo_b200_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                             unsigned cluster_z, Args&&... args) {
    return holo_launch_kernel_cluster(ctx, kernel, grid, block, smem, 1u, cluster_z, static_cast<Args&&>(args)...);
}
#endif

// ---- kernel launchers (each validates nothing: geometry is checked by the dispatcher) ------
// lut.cu
int32_t holo_lut_table(holo_b200_ctx* ctx, uint8_t act, uint8_t dtype, const uint16_t** table);
int32_t holo_launch_lut(holo_b200_ctx* ctx, const uint16_t* table, const uint16_t* in, uint16_t* out, uint64_t n);
// glue.cu
// the elementwise variants served as one exact IEEE operation per element (beyond Add / Mul and the LUT activations)
inline bool holo_is_exact_unary(uint32_t k) {
    return k == HOLO_K_NEG || k == HOLO_K_RELU || k == HOLO_K_SQRT || k == HOLO_K_RECIPROCAL || k == HOLO_K_CEIL || k == HOLO_K_FLOOR ||
           k == HOLO_K_ROUND || k == HOLO_K_IS_NAN || k == HOLO_K_SIGN || k == HOLO_K_ABS;
}
inline bool holo_is_exact_binary(uint32_t k) {
    return k == HOLO_K_SUB || k == HOLO_K_DIV || k == HOLO_K_MOD || (k >= HOLO_K_MIN && k <= HOLO_K_GREATER_OR_EQUAL);
}
int32_t holo_launch_elementwise(holo_b200_ctx* ctx, int tag, const void* a, const void* b, void* out, uint64_t n, uint8_t dtype);
int32_t holo_launch_binary(holo_b200_ctx* ctx, int op, const void* a, const void* b, void* out, uint64_t n, uint8_t dtype);
int32_t holo_launch_rms_norm(holo_b200_ctx* ctx, const void* x, const void* residual, const void* gamma, void* out,
                             uint32_t batch, uint32_t feature, float eps, uint8_t dtype);
int32_t holo_launch_rope_quantize(holo_b200_ctx* ctx, const void* x, const void* c, const void* s, void* rope_out, int8_t* codes,
                                  float* scales, uint64_t rows, uint32_t d, uint8_t dtype);
int32_t holo_launch_layer_norm(holo_b200_ctx* ctx, const void* x, const void* gamma, const void* beta, void* out, uint32_t batch,
                               uint32_t feature, float eps, uint8_t dtype);
int32_t holo_launch_broadcast(holo_b200_ctx* ctx, const uint8_t* small, const uint8_t* other, uint8_t* out, uint32_t rank,
                              const uint32_t* in_dims, const uint32_t* out_dims, uint32_t es, int op, int small_is_lhs, uint8_t dtype);
int32_t holo_launch_where(holo_b200_ctx* ctx, const uint8_t* cond, const void* a, const void* b, void* out, uint64_t n, uint8_t dtype);
int32_t holo_launch_dequant_activation(holo_b200_ctx* ctx, const uint8_t* in, float* out, uint64_t n, uint8_t quant_dtype, uint8_t act,
                                       float scale, int32_t zero_point);
int32_t holo_launch_reduce(holo_b200_ctx* ctx, const void* in, void* out, uint32_t rank, const uint32_t* dims, uint32_t axes_mask,
                           uint64_t n, int kind, int mean, uint8_t dtype);
int32_t holo_launch_softmax(holo_b200_ctx* ctx, const void* x, void* out, uint32_t batch, uint32_t feature, uint8_t dtype);
int32_t holo_launch_transpose(holo_b200_ctx* ctx, const uint8_t* in, uint8_t* out, uint32_t rank, const uint32_t* dims,
                              const uint8_t* perm, uint32_t es);
int32_t holo_launch_rope(holo_b200_ctx* ctx, const void* x, const void* c, const void* s, void* out, uint32_t head_dim,
                         uint64_t n, uint8_t dtype);
int32_t holo_launch_gather(holo_b200_ctx* ctx, const uint8_t* data, const void* idx, uint8_t idx_dtype, uint8_t* out,
                           uint64_t outer, uint64_t axis_dim, uint64_t inner_bytes, uint64_t num_idx);
int32_t holo_launch_cast(holo_b200_ctx* ctx, const void* in, uint8_t src, void* out, uint8_t dst, uint64_t n);
int32_t holo_launch_dequantize(holo_b200_ctx* ctx, const HoloDequantizeCall& c, const void* in, const float* scales,
                               const int32_t* zps, void* out);
int32_t holo_launch_kv_write(holo_b200_ctx* ctx, const uint8_t* cache, const uint8_t* newr, const uint32_t* pos,
                             uint8_t* out, uint32_t planes, uint32_t bucket, uint32_t new_rows, uint32_t row_bytes);
int32_t holo_launch_quantize_rows(holo_b200_ctx* ctx, const void* x, uint8_t dtype, uint64_t rows, uint32_t d,
                                  int8_t* codes, float* scales);
int32_t holo_launch_micro_batch(holo_b200_ctx* ctx, const HoloMicroOp* dev_ops, uint32_t nops, uint32_t total_ctas);
// attention.cu
struct HoloAttnArgs {
    const void* q;
    const void *k_past, *v_past, *k_new, *v_new;              // bf16/f16/f32 rows, or i8 codes when quantized
    const float *k_past_s, *v_past_s, *k_new_s, *v_new_s;     // per-row scales (quantized form only)
    const uint32_t* valid_len;   // scalar-mask form; null = every cache row is visible
    const float* mask;           // additive-mask form ([m, past + nnew] f32) when non-null: every key takes part
    void* out;
    uint32_t b, h, hkv, m, past, nnew, d;
    float scale_div;  // scores are divided by this
    uint8_t dtype;    // q / out dtype (and KV dtype in the unquantized form)
    bool quantized;
    bool all_new;     // scalar-mask form without the causal law: query row i sees every chunk row (legacy non-causal Attention)
};
int32_t holo_launch_decode_attention(holo_b200_ctx* ctx, const HoloAttnArgs& a);
// gemm.cu
int32_t holo_launch_matmul(holo_b200_ctx* ctx, const void* a, const void* b, void* out, uint32_t m, uint32_t k,
                           uint32_t n, uint8_t dtype, uint8_t fused_act, const void* residual, bool b_constant = false);
// One column segment of a merged matmul: `width` columns of the product go to `out`
// ([m, width] row-major) through their own epilogue.
struct HoloMatmulSeg {
    void* out;
    const void* residual;
    uint32_t width;
    uint8_t fused_act;
    // 1: the product has 2 * width columns laid out as alternating 64-column blocks of a "gate" and an
    // "up" projection; out[:, j] = narrow(widen(act(narrow(gate_j))) * widen(narrow(up_j))) (the
    // MatMulActivation -> Mul pair of a gated FFN in one epilogue). Single segment only.
    uint8_t gated = 0;
    // 1: the product is a partial of a tensor-parallel sum: out = narrow(sum over ranks of
    // narrow(A . B)) (+ residual), the exchange done by the matmul's own epilogue over peer memory
    // when the group has the peer-memory transport, by a following all-reduce launch otherwise
    uint8_t all_reduce = 0;
    // Work on the stored [m, width] values by heads of 128 columns, done by the product's own epilogue in place
    // of the calls that would read `out`: 1 = RotaryEmbedding (head_dim 128; cos / sin laid out like out) into
    // rope_out; 2 = that, then QuantizeRowsI8 of the rotated rows (one row per head) into codes / scales;
    // 3 = QuantizeRowsI8 of the stored rows. `out` is still written. See holo_matmul_head_ops_ok.
    uint8_t head_op = 0;
    // 1 (first segment speaks for the product): B is a constant weight that no launch of the stream writes, so
    // the kernel may request its first tiles before it waits for the previous kernel
    uint8_t b_constant = 0;
    const void* cos = nullptr;
    const void* sin = nullptr;
    void* rope_out = nullptr;
    int8_t* codes = nullptr;
    float* scales = nullptr;
};
bool holo_matmul_head_ops_ok(uint32_t m, uint32_t k, uint32_t n, uint8_t dtype, const HoloMatmulSeg* segs, uint32_t nseg);
// act(A . B + residual) on the exact per-cell kernel (MatMulAddActivation)
int32_t holo_launch_matmul_add_activation(holo_b200_ctx* ctx, const void* a, const void* b, void* out, uint32_t m, uint32_t k, uint32_t n,
                                          uint8_t dtype, uint8_t fused_act, const void* residual);
int32_t holo_launch_matmul_multi(holo_b200_ctx* ctx, const void* a, const void* b, uint32_t m, uint32_t k, uint32_t n,
                                 uint8_t dtype, const HoloMatmulSeg* segs, uint32_t nseg);
// quant_gemv.cu
int32_t holo_launch_matmul_e8cb_omajor(holo_b200_ctx* ctx, const float* a, const uint8_t* bq, const int8_t* codebook, const float* scales,
                                       const int32_t* zero_points, const float* residual, float* out, uint32_t m, uint32_t k, uint32_t n, int act);
int32_t holo_launch_matmul_w8a8_omajor(holo_b200_ctx* ctx, const float* a, const int8_t* bq, const float* scales, const int32_t* zero_points,
                                       const float* residual, float* out, uint32_t m, uint32_t k, uint32_t n, int act, bool i4);
int32_t holo_launch_matmul_dequant_kn(holo_b200_ctx* ctx, const float* a, const uint8_t* bq, const float* scales, const int32_t* zero_points,
                                      const float* residual, float* out, uint32_t m, uint32_t k, uint32_t n, uint32_t channels, uint32_t inner,
                                      uint8_t quant_dtype, float scale, int32_t zero_point, int act);
// tp.cu
int32_t holo_all_reduce(holo_b200_ctx* ctx, void* buf, uint64_t n, uint8_t dtype);
int32_t holo_all_reduce_add(holo_b200_ctx* ctx, const void* partial, const void* residual, void* out, uint64_t n, uint8_t dtype);
void holo_tp_destroy(holo_b200_ctx* ctx);
