// Decoder glue ops: the small HBM-bound kernels around the three hot families.
// Each replaces one CPU kernel of crates/hologram-compute/src/cpu (cited per kernel).
// Elementwise arithmetic uses explicit round-to-nearest intrinsics in the reference's
// evaluation order, so Add / Mul / RoPE / Cast / Dequantize / the row quantizer are
// bit-identical to the CPU path; RMSNorm reduces its sum of squares in parallel and is
// therefore a tolerance-class op.
#include "common.h"
#include "numerics.cuh"

namespace {

constexpr int EW_THREADS = 256;
inline unsigned ew_blocks(uint64_t n, int per_thread = 1) {
    uint64_t b = (n + (uint64_t)EW_THREADS * per_thread - 1) / ((uint64_t)EW_THREADS * per_thread);
    if (b < 1) b = 1;
    if (b > 1u << 20) b = 1u << 20;
    return (unsigned)b;
}

// binary_float_acc, cpu/float_kernels.rs:252-296: widen, op, narrow.
__device__ __forceinline__ void binary_body(int op, const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out,
                                            uint64_t n, int dtype, uint32_t block, uint32_t nblocks) {
    uint64_t stride = (uint64_t)nblocks * blockDim.x;
    for (uint64_t i = (uint64_t)block * blockDim.x + threadIdx.x; i < n; i += stride) {
        float va = holo::load_float(a, i, dtype), vb = holo::load_float(b, i, dtype);
        holo::store_float(out, i, op == 0 ? __fadd_rn(va, vb) : __fmul_rn(va, vb), dtype);
    }
}

__global__ void binary_kernel(int op, const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out,
                              uint64_t n, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    binary_body(op, a, b, out, n, dtype, blockIdx.x, gridDim.x);
}

// The exact elementwise forms beyond Add / Mul and the LUT activations (unary_float and binary_float,
// cpu/float_kernels.rs:190-233, :236-296): widen, one IEEE operation, narrow; `tag` is the wire discriminant.
__global__ void elementwise_kernel(int tag, const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out,
                                   uint64_t n, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool unary = holo::ew_is_unary(tag);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float va = holo::load_float(a, i, dtype);
        holo::store_float(out, i, unary ? holo::ew_unary(tag, va) : holo::ew_binary(tag, va, holo::load_float(b, i, dtype)), dtype);
    }
}

// 16-bit fast path: eight elements per thread through 128-bit loads and stores.
__device__ __forceinline__ void binary16_vec_body(int op, const uint4* __restrict__ a, const uint4* __restrict__ b,
                                                  uint4* __restrict__ out, uint64_t nvec, int dtype, uint32_t block, uint32_t nblocks) {
    uint64_t stride = (uint64_t)nblocks * blockDim.x;
    for (uint64_t i = (uint64_t)block * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        uint4 va = a[i], vb = b[i], r;
        const uint32_t* pa = &va.x;
        const uint32_t* pb = &vb.x;
        uint32_t* pr = &r.x;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float a0 = holo::widen16((uint16_t)(pa[w] & 0xffffu), dtype), a1 = holo::widen16((uint16_t)(pa[w] >> 16), dtype);
            float b0 = holo::widen16((uint16_t)(pb[w] & 0xffffu), dtype), b1 = holo::widen16((uint16_t)(pb[w] >> 16), dtype);
            float r0 = op == 0 ? __fadd_rn(a0, b0) : __fmul_rn(a0, b0);
            float r1 = op == 0 ? __fadd_rn(a1, b1) : __fmul_rn(a1, b1);
            pr[w] = (uint32_t)holo::narrow16(r0, dtype) | ((uint32_t)holo::narrow16(r1, dtype) << 16);
        }
        out[i] = r;
    }
}
__global__ void binary16_vec_kernel(int op, const uint4* __restrict__ a, const uint4* __restrict__ b,
                                    uint4* __restrict__ out, uint64_t nvec, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    binary16_vec_body(op, a, b, out, nvec, dtype, blockIdx.x, gridDim.x);
}

// rms_norm_float, cpu/float_kernels.rs:1683-1756: inv = 1/sqrt(sumsq/f + eps),
// out = x * inv * gamma (left to right). One CTA per row.
// With `residual` (add_rms_norm_float, :1567-1681) the row is x + residual, summed in f32 and not
// narrowed before the norm.
__global__ void rms_norm_kernel(const void* __restrict__ x, const void* __restrict__ residual, const void* __restrict__ gamma,
                                void* __restrict__ out, uint32_t feature, float eps, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    __shared__ float s_part[32];
    __shared__ float s_inv;
    const uint64_t off = (uint64_t)blockIdx.x * feature;
    float acc = 0.0f;
    for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x) {
        float v = holo::load_float(x, off + j, dtype);
        if (residual) v = __fadd_rn(v, holo::load_float(residual, off + j, dtype));
        acc = fmaf(v, v, acc);
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.0f;
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)feature), eps)));
    }
    __syncthreads();
    const float inv = s_inv;
    for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x) {
        float g = gamma ? holo::load_float(gamma, j, dtype) : 1.0f;
        float xv = holo::load_float(x, off + j, dtype);
        if (residual) xv = __fadd_rn(xv, holo::load_float(residual, off + j, dtype));
        float v = __fmul_rn(__fmul_rn(xv, inv), g);
        holo::store_float(out, off + j, v, dtype);
    }
}

// 16-bit rows with feature % 8 == 0 and feature <= 8192: one pass, eight elements per thread
// held in registers between the reduction and the scaling.
__global__ void __launch_bounds__(1024)
rms_norm16_vec_kernel(const uint4* __restrict__ x, const uint4* __restrict__ residual, const uint4* __restrict__ gamma,
                      uint4* __restrict__ out, uint32_t feature, float eps, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    __shared__ float s_part[32];
    __shared__ float s_inv;
    const uint32_t nvec = feature >> 3;
    const uint64_t off = (uint64_t)blockIdx.x * nvec;
    const bool active = threadIdx.x < nvec;
    float v[8];
    float acc = 0.0f;
    uint4 g = make_uint4(0, 0, 0, 0);
    if (active) {
        if (gamma) g = gamma[threadIdx.x];   // requested with the row, not after the reduction: one round trip less
        uint4 w = x[off + threadIdx.x];
        const uint32_t* pw = &w.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = holo::widen16((uint16_t)(pw[i] & 0xffffu), dtype);
            v[2 * i + 1] = holo::widen16((uint16_t)(pw[i] >> 16), dtype);
        }
        if (residual) {
            uint4 rw = residual[off + threadIdx.x];
            const uint32_t* pr = &rw.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __fadd_rn(v[2 * i], holo::widen16((uint16_t)(pr[i] & 0xffffu), dtype));
                v[2 * i + 1] = __fadd_rn(v[2 * i + 1], holo::widen16((uint16_t)(pr[i] >> 16), dtype));
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(v[i], v[i], acc);
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.0f;
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)feature), eps)));
    }
    __syncthreads();
    if (!active) return;
    const float inv = s_inv;
    const uint32_t* pg = &g.x;
    uint4 r;
    uint32_t* pr = &r.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float g0 = gamma ? holo::widen16((uint16_t)(pg[i] & 0xffffu), dtype) : 1.0f;
        float g1 = gamma ? holo::widen16((uint16_t)(pg[i] >> 16), dtype) : 1.0f;
        float r0 = __fmul_rn(__fmul_rn(v[2 * i], inv), g0), r1 = __fmul_rn(__fmul_rn(v[2 * i + 1], inv), g1);
        pr[i] = (uint32_t)holo::narrow16(r0, dtype) | ((uint32_t)holo::narrow16(r1, dtype) << 16);
    }
    out[off + threadIdx.x] = r;
}

// transpose_float, cpu/float_kernels.rs:2980-3027: output axis i is input axis perm[i]; every
// output element is gathered from its permuted input position (element size 1, 2, 4 or 8 bytes).
struct TransposeParams {
    uint32_t out_dims[8];
    uint64_t in_strides_perm[8];   // stride (in elements) of the input axis feeding output axis i
    uint32_t rank, es;
    uint64_t total;
};
__global__ void transpose_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, const TransposeParams p) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; o < p.total; o += stride) {
        uint64_t rem = o, src = 0;
        for (int i = (int)p.rank - 1; i >= 0; --i) {
            const uint32_t c = (uint32_t)(rem % p.out_dims[i]);
            rem /= p.out_dims[i];
            src += (uint64_t)c * p.in_strides_perm[i];
        }
        switch (p.es) {
            case 1: out[o] = in[src]; break;
            case 2: reinterpret_cast<uint16_t*>(out)[o] = reinterpret_cast<const uint16_t*>(in)[src]; break;
            case 4: reinterpret_cast<uint32_t*>(out)[o] = reinterpret_cast<const uint32_t*>(in)[src]; break;
            default: reinterpret_cast<uint64_t*>(out)[o] = reinterpret_cast<const uint64_t*>(in)[src]; break;
        }
    }
}

// where_float, cpu/float_kernels.rs:2908-2937: a byte of condition per element picks a or b; the value goes
// through the dtype's read and write as on the CPU (an f16 NaN comes out as the one quiet pattern).
__global__ void where_kernel(const uint8_t* __restrict__ cond, const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out,
                             uint64_t n, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        holo::store_float(out, i, cond[i] != 0 ? holo::load_float(a, i, dtype) : holo::load_float(b, i, dtype), dtype);
}

// dequant_activation, cpu/kernels.rs:311-381: the composition activation((q - zp) * scale) has at most 256
// distinct inputs, so every CTA builds the table of all of them in shared memory (one entry per thread,
// the same f32 arithmetic and scalar activation as dequantize followed by the unary call) and then
// streams: 1 byte in, 4 bytes out per element (i4: two elements per byte, low nibble first).
__global__ void __launch_bounds__(256)
dequant_activation_kernel(const uint8_t* __restrict__ in, float* __restrict__ out, uint64_t n, int quant_dtype, int act, float scale, int zp) {
    holo_pdl_trigger();
    holo_pdl_wait();
    __shared__ float s_table[256];
    {
        const int raw = threadIdx.x;
        int q = raw;
        if (quant_dtype == HOLO_DTYPE_I8) q = (int)(int8_t)raw;
        else if (quant_dtype == HOLO_DTYPE_I4) q = (raw & 15) >= 8 ? (raw & 15) - 16 : (raw & 15);
        s_table[raw] = holo::lut_act_ref(act, __fmul_rn(__int2float_rn(q - zp), scale));
    }
    __syncthreads();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, t0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (quant_dtype == HOLO_DTYPE_I4) {
        for (uint64_t b = t0; b < (n + 1) / 2; b += stride) {
            const uint8_t byte = in[b];
            out[2 * b] = s_table[byte & 15];
            if (2 * b + 1 < n) out[2 * b + 1] = s_table[byte >> 4];
        }
        return;
    }
    const bool vec = (((uintptr_t)in | (uintptr_t)out) & 15u) == 0;
    const uint64_t nvec = vec ? n >> 4 : 0;
    for (uint64_t v = t0; v < nvec; v += stride) {
        const uint4 w = reinterpret_cast<const uint4*>(in)[v];
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
            reinterpret_cast<float4*>(out)[v * 4 + j] = make_float4(s_table[words[j] & 255u], s_table[(words[j] >> 8) & 255u],
                                                                    s_table[(words[j] >> 16) & 255u], s_table[words[j] >> 24]);
    }
    for (uint64_t i = (nvec << 4) + t0; i < n; i += stride) out[i] = s_table[in[i]];
}

// reduce_float, cpu/float_kernels.rs:1901-2022 (ReducePlan :2024-2099). kind 0 sum, 1 prod, 2 min, 3 max.
struct ReduceParams {
    uint32_t kept_dims[8], red_dims[8];
    uint64_t kept_strides[8], red_strides[8];   // input strides (elements) of the kept and of the reduced axes
    uint32_t n_kept, n_red;
    uint64_t out_count, reduced_count;
    int kind, mean, dtype;
};
__device__ __forceinline__ float reduce_fold(int kind, float a, float b) {
    return kind == 0 ? __fadd_rn(a, b) : kind == 1 ? __fmul_rn(a, b) : kind == 2 ? holo::min_ref(a, b) : holo::max_ref(a, b);
}
__device__ __forceinline__ float reduce_init(int kind) { return kind == 0 ? 0.0f : kind == 1 ? 1.0f : kind == 2 ? INFINITY : -INFINITY; }

// One thread per output cell, folding the cell's inputs in linear input order; with a 16-bit dtype the
// running value is narrowed after every step, as the CPU loop keeps it in the output buffer.
__global__ void reduce_cells_kernel(const void* __restrict__ in, void* __restrict__ out, const ReduceParams p) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= p.out_count) return;
    uint64_t rem = o, base = 0;
    for (int i = (int)p.n_kept - 1; i >= 0; --i) {
        base += (rem % p.kept_dims[i]) * p.kept_strides[i];
        rem /= p.kept_dims[i];
    }
    const bool narrow = p.dtype != HOLO_DTYPE_F32;
    float acc = reduce_init(p.kind);
    if (narrow) acc = holo::widen16(holo::narrow16(acc, p.dtype), p.dtype);
    uint32_t coord[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint64_t off = base;
    for (uint64_t r = 0; r < p.reduced_count; ++r) {
        acc = reduce_fold(p.kind, acc, holo::load_float(in, off, p.dtype));
        if (narrow) acc = holo::widen16(holo::narrow16(acc, p.dtype), p.dtype);
        for (int a = (int)p.n_red - 1; a >= 0; --a) {   // odometer over the reduced axes, rightmost fastest
            off += p.red_strides[a];
            if (++coord[a] < p.red_dims[a]) break;
            off -= p.red_strides[a] * p.red_dims[a];
            coord[a] = 0;
        }
    }
    if (p.mean) {
        acc = __fmul_rn(acc, __fdiv_rn(1.0f, (float)p.reduced_count));
    }
    holo::store_float(out, o, acc, p.dtype);
}

// Full f32 reduction to one cell (sum, min, max): one CTA, tree order (the CPU folds in SIMD chunks here,
// so the sum agrees to rounding; min and max are order-independent).
__global__ void reduce_all_f32_kernel(const float* __restrict__ in, float* __restrict__ out, uint64_t n, int kind, int mean) {
    holo_pdl_trigger();
    holo_pdl_wait();
    __shared__ float s_part[32];
    float acc = reduce_init(kind);
    for (uint64_t i = threadIdx.x; i < n; i += blockDim.x) acc = reduce_fold(kind, acc, in[i]);
    for (int o = 16; o > 0; o >>= 1) acc = reduce_fold(kind, acc, __shfl_xor_sync(0xffffffffu, acc, o));
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = s_part[0];
        for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) t = reduce_fold(kind, t, s_part[w]);
        out[0] = mean ? __fdiv_rn(t, (float)n) : t;
    }
}

// expand_float and broadcast_binary_float (cpu/float_kernels.rs:3405-3444, :3250-3397): every output element
// reads the small operand at the row-major index built from its coordinates with stride 0 on the
// broadcast axes. op < 0: a plain copy of `es` bytes (Expand); otherwise one f32 operation on the
// widened operands, narrowed once (bit-identical to the CPU loop).
struct BroadcastParams {
    uint32_t out_dims[8];
    uint64_t in_strides[8];
    uint32_t rank, es;
    uint64_t total;
    int op, small_is_lhs, dtype;
};
__global__ void broadcast_kernel(const uint8_t* __restrict__ small, const uint8_t* __restrict__ other, uint8_t* __restrict__ out,
                                 const BroadcastParams p) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; o < p.total; o += stride) {
        uint64_t rem = o, idx = 0;
        for (int i = (int)p.rank - 1; i >= 0; --i) {
            idx += (rem % p.out_dims[i]) * p.in_strides[i];
            rem /= p.out_dims[i];
        }
        if (p.op < 0) {
            if (p.es == 4) reinterpret_cast<uint32_t*>(out)[o] = reinterpret_cast<const uint32_t*>(small)[idx];
            else if (p.es == 2) reinterpret_cast<uint16_t*>(out)[o] = reinterpret_cast<const uint16_t*>(small)[idx];
            else for (uint32_t b = 0; b < p.es; ++b) out[o * p.es + b] = small[idx * p.es + b];
        } else {
            const float sv = holo::load_float(small, idx, p.dtype), ov = holo::load_float(other, o, p.dtype);
            const float a = p.small_is_lhs ? sv : ov, b = p.small_is_lhs ? ov : sv;
            const float r = p.op == 0 ? __fadd_rn(a, b) : p.op == 1 ? __fsub_rn(a, b) : __fmul_rn(a, b);
            holo::store_float(out, o, r, p.dtype);
        }
    }
}

// layer_norm_float, cpu/float_kernels.rs:1338-1445: mean, variance of the centred row, inv = 1/sqrt(var + eps),
// out = (x - mean) * inv * gamma + beta (absent gamma = 1, absent beta = 0). One CTA per row; the two
// sums are reduced in parallel (the CPU sums left to right), so results agree to rounding of the sums.
__device__ __forceinline__ float block_sum(float v, float* s_part, float* s_val) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) s_part[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (uint32_t w = 0; w < nw; ++w) t = __fadd_rn(t, s_part[w]);
        *s_val = t;
    }
    __syncthreads();
    return *s_val;
}

__global__ void layer_norm_kernel(const void* __restrict__ x, const void* __restrict__ gamma, const void* __restrict__ beta,
                                  void* __restrict__ out, uint32_t feature, float eps, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    __shared__ float s_part[32];
    __shared__ float s_val;
    const uint64_t off = (uint64_t)blockIdx.x * feature;
    float sum = 0.0f;
    for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x) sum = __fadd_rn(sum, holo::load_float(x, off + j, dtype));
    const float mean = __fdiv_rn(block_sum(sum, s_part, &s_val), (float)feature);
    float sq = 0.0f;
    for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x) {
        const float d = __fsub_rn(holo::load_float(x, off + j, dtype), mean);
        sq = __fadd_rn(sq, __fmul_rn(d, d));
    }
    const float var = __fdiv_rn(block_sum(sq, s_part, &s_val), (float)feature);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x) {
        const float g = gamma ? holo::load_float(gamma, j, dtype) : 1.0f;
        const float b = beta ? holo::load_float(beta, j, dtype) : 0.0f;
        const float d = __fsub_rn(holo::load_float(x, off + j, dtype), mean);
        holo::store_float(out, off + j, __fadd_rn(__fmul_rn(__fmul_rn(d, inv), g), b), dtype);
    }
}

// softmax_float, cpu/float_kernels.rs:1758-1875: m = max, e_j = exp_det(x_j - m), out_j = e_j / max(sum, 1e-30);
// a row whose maximum is -inf is all zeros. One CTA per row; the sum is reduced in parallel (the CPU
// sums left to right), so results agree to rounding of the sum, not bit for bit.
__global__ void softmax_kernel(const void* __restrict__ x, void* __restrict__ out, uint32_t feature, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    __shared__ float s_part[32];
    __shared__ float s_val;
    const uint64_t off = (uint64_t)blockIdx.x * feature;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    float mx = -INFINITY;
    for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x) {
        const float v = holo::load_float(x, off + j, dtype);
        mx = v > mx ? v : mx;       // f32::max ignores a NaN operand
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, mx, o);
        mx = other > mx ? other : mx;
    }
    if (lane == 0) s_part[warp] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = s_part[0];
        for (uint32_t w = 1; w < nw; ++w) m = s_part[w] > m ? s_part[w] : m;
        s_val = m;
    }
    __syncthreads();
    mx = s_val;
    if (mx == -INFINITY) {
        for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x) holo::store_float(out, off + j, 0.0f, dtype);
        return;
    }
    float sum = 0.0f;
    for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x)
        sum = __fadd_rn(sum, holo::exp_det(__fsub_rn(holo::load_float(x, off + j, dtype), mx)));
    for (int o = 16; o > 0; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
    __syncthreads();
    if (lane == 0) s_part[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (uint32_t w = 0; w < nw; ++w) t = __fadd_rn(t, s_part[w]);
        s_val = fmaxf(t, 1e-30f);
    }
    __syncthreads();
    const float denom = s_val;
    for (uint32_t j = threadIdx.x; j < feature; j += blockDim.x) {
        const float e = holo::exp_det(__fsub_rn(holo::load_float(x, off + j, dtype), mx));
        holo::store_float(out, off + j, __fdiv_rn(e, denom), dtype);
    }
}

// rope_float, cpu/float_kernels.rs:3123-3190 (rotate-half; cos/sin share x's layout).
__device__ __forceinline__ void rope_body(const void* __restrict__ x, const void* __restrict__ c, const void* __restrict__ s,
                                          void* __restrict__ out, uint32_t d, uint64_t n, int dtype, uint32_t block, uint32_t nblocks) {
    const uint32_t half = d >> 1;
    uint64_t stride = (uint64_t)nblocks * blockDim.x;
    for (uint64_t e = (uint64_t)block * blockDim.x + threadIdx.x; e < n; e += stride) {
        uint32_t pos = (uint32_t)(e % d);
        uint64_t base = e - pos;
        float xe = holo::load_float(x, e, dtype), ce = holo::load_float(c, e, dtype), se = holo::load_float(s, e, dtype);
        float v;
        if (pos < half) v = __fsub_rn(__fmul_rn(xe, ce), __fmul_rn(holo::load_float(x, base + pos + half, dtype), se));
        else v = __fadd_rn(__fmul_rn(xe, ce), __fmul_rn(holo::load_float(x, base + pos - half, dtype), se));
        holo::store_float(out, e, v, dtype);
    }
}
__global__ void rope_kernel(const void* __restrict__ x, const void* __restrict__ c, const void* __restrict__ s,
                            void* __restrict__ out, uint32_t d, uint64_t n, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    rope_body(x, c, s, out, d, n, dtype, blockIdx.x, gridDim.x);
}

// gather, cpu/kernels.rs:389-446: out[o,k,:] = data[o, idx[k], :]; negative indices wrap;
// an out-of-range index raises bit 0 of the status word and copies nothing.
__global__ void gather_kernel(const uint8_t* __restrict__ data, const void* __restrict__ idx, int idx_dtype,
                              uint8_t* __restrict__ out, uint64_t axis_dim, uint64_t row_bytes, uint64_t num_idx,
                              uint32_t* status) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint64_t o = blockIdx.y, k = blockIdx.x;
    long long ix = idx_dtype == HOLO_DTYPE_I32 ? (long long)((const int32_t*)idx)[k] : ((const long long*)idx)[k];
    if (ix < 0) ix += (long long)axis_dim;
    if (ix < 0 || (uint64_t)ix >= axis_dim) {
        if (threadIdx.x == 0) atomicOr(status, 1u);
        return;
    }
    const uint8_t* src = data + (o * axis_dim + (uint64_t)ix) * row_bytes;
    uint8_t* dst = out + (o * num_idx + k) * row_bytes;
    if ((((uintptr_t)src | (uintptr_t)dst | row_bytes) & 15u) == 0) {
        for (uint64_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x)
            ((uint4*)dst)[i] = ((const uint4*)src)[i];
    } else {
        for (uint64_t i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = src[i];
    }
}

// cast, cpu/kernels.rs:560-594. Float sources travel through f64 in the reference; every
// f16/bf16/f32 value is exact in f32 as well, so f32 is used as the carrier here.
__device__ __forceinline__ double load_num(const void* p, uint64_t i, int dt) {
    switch (dt) {
        case HOLO_DTYPE_F32: case HOLO_DTYPE_F16: case HOLO_DTYPE_BF16: return (double)holo::load_float(p, i, dt);
        case HOLO_DTYPE_F64: return ((const double*)p)[i];
        case HOLO_DTYPE_BOOL: case HOLO_DTYPE_U8: return (double)((const uint8_t*)p)[i];
        case HOLO_DTYPE_I8: return (double)((const int8_t*)p)[i];
        case HOLO_DTYPE_I32: return (double)((const int32_t*)p)[i];
        default: return (double)((const long long*)p)[i];
    }
}
__global__ void cast_kernel(const void* __restrict__ in, int src, void* __restrict__ out, int dst, uint64_t n) {
    holo_pdl_trigger();
    holo_pdl_wait();
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool src_f = src >= HOLO_DTYPE_F16 && src <= HOLO_DTYPE_F64;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (dst == HOLO_DTYPE_F32 || dst == HOLO_DTYPE_F16 || dst == HOLO_DTYPE_BF16) {
            holo::store_float(out, i, (float)load_num(in, i, src), dst);
        } else {
            long long v;
            if (src_f) {
                double t = trunc(load_num(in, i, src));
                // Rust `f64 as i64`: saturating, NaN -> 0
                v = t != t ? 0 : (t >= 9223372036854775808.0 ? LLONG_MAX : (t <= -9223372036854775808.0 ? LLONG_MIN : (long long)t));
            } else if (src == HOLO_DTYPE_I64 || src == HOLO_DTYPE_U64) {
                v = ((const long long*)in)[i];
            } else {
                v = (long long)load_num(in, i, src);
            }
            switch (dst) {
                case HOLO_DTYPE_BOOL: ((uint8_t*)out)[i] = v != 0; break;
                case HOLO_DTYPE_U8: ((uint8_t*)out)[i] = (uint8_t)v; break;
                case HOLO_DTYPE_I8: ((int8_t*)out)[i] = (int8_t)v; break;
                case HOLO_DTYPE_I32: ((int32_t*)out)[i] = (int32_t)v; break;
                default: ((long long*)out)[i] = v; break;
            }
        }
    }
}

// dequantize, cpu/kernels.rs:185-296: out = ((q - zp) as f32) * scale, channel = (i/inner) % channels.
__global__ void dequantize_kernel(const void* __restrict__ in, int qdt, const float* __restrict__ scales,
                                  const int32_t* __restrict__ zps, uint32_t channels, uint32_t inner, float scale,
                                  int32_t zp, void* __restrict__ out, int dtype, uint64_t n) {
    holo_pdl_trigger();
    holo_pdl_wait();
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int q = qdt == HOLO_DTYPE_I8 ? (int)((const int8_t*)in)[i] : (int)((const uint8_t*)in)[i];
        float s = scale;
        int z = zp;
        if (scales) {
            uint64_t ch = (i / inner) % channels;
            s = scales[ch];
            z = zps ? zps[ch] : 0;
        }
        holo::store_float(out, i, __fmul_rn(__int2float_rn(q - z), s), dtype);
    }
}

// kv_cache_write rows, cpu/kernels.rs:455-501: out[p][(pos + j) % bucket] = new[p][j].
// `pos` is read on the device from its 4-byte operand (no host round-trip).
__global__ void kv_write_rows_kernel(const uint8_t* __restrict__ newr, const uint32_t* __restrict__ pos,
                                     uint8_t* __restrict__ out, uint32_t bucket, uint32_t new_rows, uint32_t row_bytes) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint32_t p = blockIdx.y, j = blockIdx.x;
    const uint32_t p0 = *pos % bucket;
    const uint8_t* src = newr + ((uint64_t)p * new_rows + j) * row_bytes;
    uint8_t* dst = out + ((uint64_t)p * bucket + (p0 + j) % bucket) * row_bytes;
    if ((((uintptr_t)src | (uintptr_t)dst | row_bytes) & 15u) == 0) {
        for (uint32_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) ((uint4*)dst)[i] = ((const uint4*)src)[i];
    } else {
        for (uint32_t i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = src[i];
    }
}

// Same row copy with one warp per (plane, new row) pair, for the batched launch.
__device__ __forceinline__ void kv_write_rows_body(const uint8_t* __restrict__ newr, const uint32_t* __restrict__ pos,
                                                   uint8_t* __restrict__ out, uint32_t planes, uint32_t bucket, uint32_t new_rows,
                                                   uint32_t row_bytes, uint32_t block) {
    const uint64_t item = (uint64_t)block * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (uint64_t)planes * new_rows) return;
    const uint32_t p = (uint32_t)(item / new_rows), j = (uint32_t)(item % new_rows), lane = threadIdx.x & 31;
    const uint32_t p0 = *pos % bucket;
    const uint8_t* src = newr + ((uint64_t)p * new_rows + j) * row_bytes;
    uint8_t* dst = out + ((uint64_t)p * bucket + (p0 + j) % bucket) * row_bytes;
    if ((((uintptr_t)src | (uintptr_t)dst | row_bytes) & 15u) == 0) {
        for (uint32_t i = lane; i < row_bytes / 16; i += 32) ((uint4*)dst)[i] = ((const uint4*)src)[i];
    } else {
        for (uint32_t i = lane; i < row_bytes; i += 32) dst[i] = src[i];
    }
}

// quantize_row_i8 per row, cpu/simd.rs:4761-4785. One warp per row: max|a| by shuffles
// (max is exact in any order), inv = 127/amax, t = a*inv, r = trunc(t ± 0.5) (saturating
// cvt.rzi, NaN -> 0), clamp to ±127, scale = amax/127. A zero row gives zero codes, scale 0.
__device__ __forceinline__ void quantize_rows_body(const void* __restrict__ x, int dtype, uint64_t rows, uint32_t d,
                                                   int8_t* __restrict__ codes, float* __restrict__ scales, uint32_t block) {
    const uint64_t row = (uint64_t)block * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t off = row * d;
    float amax = 0.0f;
    for (uint32_t j = lane; j < d; j += 32) {
        float v = holo::load_float(x, off + j, dtype);
        float av = v < 0.0f ? -v : v;
        if (av > amax) amax = av;
    }
    for (int o = 16; o > 0; o >>= 1) {
        float other = __shfl_xor_sync(0xffffffffu, amax, o);
        if (other > amax) amax = other;
    }
    if (amax == 0.0f) {
        for (uint32_t j = lane; j < d; j += 32) codes[off + j] = 0;
        if (lane == 0) scales[row] = 0.0f;
        return;
    }
    const float inv = __fdiv_rn(127.0f, amax);
    for (uint32_t j = lane; j < d; j += 32) {
        float t = __fmul_rn(holo::load_float(x, off + j, dtype), inv);
        int r = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
        r = max(-127, min(127, r));
        codes[off + j] = (int8_t)r;
    }
    if (lane == 0) scales[row] = __fdiv_rn(amax, 127.0f);
}
// RoPE of one head per warp followed by quantize_row_i8 of the rotated row: exactly rope_body then
// quantize_rows_body on the narrowed values the RoPE stored. Up to 256 elements per head the narrowed
// values stay in registers (no round trip through memory between the two steps); longer rows re-read
// the warp's own stores.
__device__ __forceinline__ void rope_quantize_body(const void* __restrict__ x, const void* __restrict__ c, const void* __restrict__ s,
                                                   void* __restrict__ rope_out, int8_t* __restrict__ codes, float* __restrict__ scales,
                                                   uint64_t rows, uint32_t d, int dtype, uint32_t block) {
    const uint64_t row = (uint64_t)block * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint32_t lane = threadIdx.x & 31, half = d >> 1;
    const uint64_t off = row * d;
    constexpr int KEEP = 8;                 // 8 x 32 lanes = 256 elements
    const bool keep = d <= 32 * KEEP;
    float kept[KEEP];
#pragma unroll
    for (int i = 0; i < KEEP; ++i) kept[i] = 0.0f;
    auto rotate = [&](uint32_t j) {
        const uint64_t e = off + j;
        const float xe = holo::load_float(x, e, dtype), ce = holo::load_float(c, e, dtype), se = holo::load_float(s, e, dtype);
        float v;
        if (j < half) v = __fsub_rn(__fmul_rn(xe, ce), __fmul_rn(holo::load_float(x, e + half, dtype), se));
        else v = __fadd_rn(__fmul_rn(xe, ce), __fmul_rn(holo::load_float(x, e - half, dtype), se));
        holo::store_float(rope_out, e, v, dtype);
        return dtype == HOLO_DTYPE_F32 ? v : holo::widen16(holo::narrow16(v, dtype), dtype);   // what the store kept
    };
    if (!keep) {
        for (uint32_t j = lane; j < d; j += 32) rotate(j);
        __syncwarp();
        quantize_rows_body(rope_out, dtype, rows, d, codes, scales, block);
        return;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const uint32_t j = lane + 32 * i;
        if (j < d) {
            kept[i] = rotate(j);
            const float av = kept[i] < 0.0f ? -kept[i] : kept[i];
            if (av > amax) amax = av;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, amax, o);
        if (other > amax) amax = other;
    }
    const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(127.0f, amax);
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const uint32_t j = lane + 32 * i;
        if (j < d) {
            int r = 0;
            if (amax != 0.0f) {
                const float t = __fmul_rn(kept[i], inv);
                r = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
                r = max(-127, min(127, r));
            }
            codes[off + j] = (int8_t)r;
        }
    }
    if (lane == 0) scales[row] = amax == 0.0f ? 0.0f : __fdiv_rn(amax, 127.0f);
}
__global__ void rope_quantize_kernel(const void* __restrict__ x, const void* __restrict__ c, const void* __restrict__ s,
                                     void* __restrict__ rope_out, int8_t* __restrict__ codes, float* __restrict__ scales, uint64_t rows,
                                     uint32_t d, int dtype) {
    holo_pdl_trigger();
    holo_pdl_wait();
    rope_quantize_body(x, c, s, rope_out, codes, scales, rows, d, dtype, blockIdx.x);
}

__global__ void quantize_rows_kernel(const void* __restrict__ x, int dtype, uint64_t rows, uint32_t d,
                                     int8_t* __restrict__ codes, float* __restrict__ scales) {
    holo_pdl_trigger();
    holo_pdl_wait();
    quantize_rows_body(x, dtype, rows, d, codes, scales, blockIdx.x);
}

// d % 128 == 0, 16-bit input, 8-byte aligned rows: each lane owns 4 consecutive elements
// of every 128-element segment (one 64-bit load, one 32-bit store).
__device__ __forceinline__ void quantize_rows16_vec_body(const uint16_t* __restrict__ x, int dtype, uint64_t rows, uint32_t d,
                                                         int8_t* __restrict__ codes, float* __restrict__ scales, uint32_t block) {
    const uint64_t row = (uint64_t)block * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t off = row * d;
    const uint32_t segs = d >> 7;
    float amax = 0.0f;
    for (uint32_t s = 0; s < segs; ++s) {
        uint2 w = *reinterpret_cast<const uint2*>(x + off + s * 128 + lane * 4);
        float v[4] = {holo::widen16((uint16_t)(w.x & 0xffffu), dtype), holo::widen16((uint16_t)(w.x >> 16), dtype),
                      holo::widen16((uint16_t)(w.y & 0xffffu), dtype), holo::widen16((uint16_t)(w.y >> 16), dtype)};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float av = v[e] < 0.0f ? -v[e] : v[e];
            if (av > amax) amax = av;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        float other = __shfl_xor_sync(0xffffffffu, amax, o);
        if (other > amax) amax = other;
    }
    const bool zero = amax == 0.0f;
    const float inv = zero ? 0.0f : __fdiv_rn(127.0f, amax);
    for (uint32_t s = 0; s < segs; ++s) {
        uint32_t packed = 0;
        if (!zero) {
            uint2 w = *reinterpret_cast<const uint2*>(x + off + s * 128 + lane * 4);
            float v[4] = {holo::widen16((uint16_t)(w.x & 0xffffu), dtype), holo::widen16((uint16_t)(w.x >> 16), dtype),
                          holo::widen16((uint16_t)(w.y & 0xffffu), dtype), holo::widen16((uint16_t)(w.y >> 16), dtype)};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float t = __fmul_rn(v[e], inv);
                int r = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
                r = max(-127, min(127, r));
                packed |= ((uint32_t)r & 0xffu) << (8 * e);
            }
        }
        *reinterpret_cast<uint32_t*>(codes + off + s * 128 + lane * 4) = packed;
    }
    if (lane == 0) scales[row] = zero ? 0.0f : __fdiv_rn(amax, 127.0f);
}
__global__ void quantize_rows16_vec_kernel(const uint16_t* __restrict__ x, int dtype, uint64_t rows, uint32_t d,
                                           int8_t* __restrict__ codes, float* __restrict__ scales) {
    holo_pdl_trigger();
    holo_pdl_wait();
    quantize_rows16_vec_body(x, dtype, rows, d, codes, scales, blockIdx.x);
}

// Several independent small ops in one launch: each CTA looks up the op that owns its block
// index and runs that op's body with a block index local to the op. Used by the session for
// runs of mutually independent glue calls (the trailing KV appends of all layers, the RoPE
// pair, the K/V quantizer pair), whose individual launches cost more than their work.
__global__ void __launch_bounds__(256) micro_batch_kernel(const HoloMicroOp* __restrict__ ops, uint32_t nops) {
    holo_pdl_trigger();
    holo_pdl_wait();
    // which op owns this CTA: up to 32 ops are looked at by one lane each (one round trip to the descriptors
    // instead of a chain of dependent loads); the ops' CTA ranges are ascending
    uint32_t oi = 0;
    if (nops <= 32) {
        const uint32_t lane = threadIdx.x & 31;
        const uint32_t end = lane < nops ? ops[lane].cta_begin + ops[lane].cta_count : 0xffffffffu;
        oi = __popc(__ballot_sync(0xffffffffu, blockIdx.x >= end));
        if (oi >= nops) oi = nops - 1;
    } else {
        while (oi + 1 < nops && blockIdx.x >= ops[oi].cta_begin + ops[oi].cta_count) ++oi;
    }
    const HoloMicroOp op = ops[oi];
    const uint32_t block = blockIdx.x - op.cta_begin;
    switch (op.kind) {
        case HOLO_MICRO_KV_WRITE:
            kv_write_rows_body((const uint8_t*)op.p0, (const uint32_t*)op.p1, (uint8_t*)op.o0, op.a, op.b, op.c, op.d, block);
            break;
        case HOLO_MICRO_ROPE:
            rope_body(op.p0, op.p1, op.p2, op.o0, op.a, op.n, (int)op.dtype, block, op.cta_count);
            break;
        case HOLO_MICRO_QUANT_VEC:
            quantize_rows16_vec_body((const uint16_t*)op.p0, (int)op.dtype, op.n, op.a, (int8_t*)op.o0, (float*)op.o1, block);
            break;
        case HOLO_MICRO_QUANT:
            quantize_rows_body(op.p0, (int)op.dtype, op.n, op.a, (int8_t*)op.o0, (float*)op.o1, block);
            break;
        case HOLO_MICRO_ROPE_QUANT:
            rope_quantize_body(op.p0, op.p1, op.p2, op.o0, (int8_t*)op.o1, (float*)op.o2, op.n, op.a, (int)op.dtype, block);
            break;
        case HOLO_MICRO_BINARY_VEC:
            binary16_vec_body((int)op.a, (const uint4*)op.p0, (const uint4*)op.p1, (uint4*)op.o0, op.n, (int)op.dtype, block, op.cta_count);
            break;
        default:
            binary_body((int)op.a, op.p0, op.p1, op.o0, op.n, (int)op.dtype, block, op.cta_count);
            break;
    }
}

}  // namespace

int32_t holo_launch_micro_batch(holo_b200_ctx* ctx, const HoloMicroOp* dev_ops, uint32_t nops, uint32_t total_ctas) {
    if (nops == 0 || total_ctas == 0) return HOLO_OK;
    HOLO_CUDA(holo_launch_kernel(ctx, micro_batch_kernel, dim3(total_ctas), dim3(256), 0, 1, dev_ops, nops));
    HOLO_CUDA(cudaGetLastError());
    ctx->launches++;
    return HOLO_OK;
}

// While a session records a batch, launchers append a descriptor instead of launching.
static bool record_op(holo_b200_ctx* ctx, HoloMicroOp op, uint64_t ctas) {
    if (!ctx->record) return false;
    if (ctas == 0 || ctas > 0x7fffffffull) {
        ctx->record_failed = true;
        return true;
    }
    op.cta_begin = 0;
    op.cta_count = (uint32_t)ctas;
    ctx->record->push_back(op);
    return true;
}

#define LAUNCH_CHECK(ctx)                 \
    do {                                  \
        HOLO_CUDA(cudaGetLastError());    \
        (ctx)->launches++;                \
    } while (0)

int32_t holo_launch_binary(holo_b200_ctx* ctx, int op, const void* a, const void* b, void* out, uint64_t n, uint8_t dtype) {
    if (n == 0) return HOLO_OK;
    const bool aligned = (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15u) == 0;
    if (ctx->record) {
        HoloMicroOp m = {};
        const bool vec = dtype != HOLO_DTYPE_F32 && aligned && (n % 8) == 0;
        m.kind = vec ? HOLO_MICRO_BINARY_VEC : HOLO_MICRO_BINARY;
        m.p0 = a; m.p1 = b; m.o0 = out; m.a = (uint32_t)op; m.dtype = dtype; m.n = vec ? n / 8 : n;
        record_op(ctx, m, ew_blocks(m.n));
        return HOLO_OK;
    }
    if (dtype != HOLO_DTYPE_F32 && aligned && (n % 8) == 0) {
        HOLO_CUDA(holo_launch_kernel(ctx, binary16_vec_kernel, dim3(ew_blocks(n / 8)), dim3(EW_THREADS), 0, 1, op, (const uint4*)a, (const uint4*)b,
                                                                             (uint4*)out, n / 8, dtype));
    } else {
        HOLO_CUDA(holo_launch_kernel(ctx, binary_kernel, dim3(ew_blocks(n)), dim3(EW_THREADS), 0, 1, op, a, b, out, n, dtype));
    }
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_elementwise(holo_b200_ctx* ctx, int tag, const void* a, const void* b, void* out, uint64_t n, uint8_t dtype) {
    if (n == 0) return HOLO_OK;
    HOLO_CUDA(holo_launch_kernel(ctx, elementwise_kernel, dim3(ew_blocks(n)), dim3(EW_THREADS), 0, 1, tag, a, b, out, n, (int)dtype));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_rms_norm(holo_b200_ctx* ctx, const void* x, const void* residual, const void* gamma, void* out, uint32_t batch,
                             uint32_t feature, float eps, uint8_t dtype) {
    if (batch == 0 || feature == 0) return HOLO_OK;
    const bool vec = dtype != HOLO_DTYPE_F32 && (feature % 8) == 0 && feature <= 8192 &&
                     (((uintptr_t)x | (uintptr_t)residual | (uintptr_t)gamma | (uintptr_t)out) & 15u) == 0;
    if (vec) {
        uint32_t threads = ((feature / 8 + 31) / 32) * 32;
        HOLO_CUDA(holo_launch_kernel(ctx, rms_norm16_vec_kernel, dim3(batch), dim3(threads), 0, 1, (const uint4*)x, (const uint4*)residual,
                                     (const uint4*)gamma, (uint4*)out, feature, eps, (int)dtype));
    } else {
        HOLO_CUDA(holo_launch_kernel(ctx, rms_norm_kernel, dim3(batch), dim3(256), 0, 1, x, residual, gamma, out, feature, eps, (int)dtype));
    }
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_where(holo_b200_ctx* ctx, const uint8_t* cond, const void* a, const void* b, void* out, uint64_t n, uint8_t dtype) {
    if (n == 0) return HOLO_OK;
    HOLO_CUDA(holo_launch_kernel(ctx, where_kernel, dim3(ew_blocks(n)), dim3(EW_THREADS), 0, 1, cond, a, b, out, n, (int)dtype));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_dequant_activation(holo_b200_ctx* ctx, const uint8_t* in, float* out, uint64_t n, uint8_t quant_dtype, uint8_t act,
                                       float scale, int32_t zero_point) {
    if (n == 0) return HOLO_OK;
    const uint64_t units = quant_dtype == HOLO_DTYPE_I4 ? (n + 1) / 2 : (n + 15) / 16;
    const uint64_t want = (units + 255) / 256, cap = (uint64_t)ctx->sm_count * 8;
    HOLO_CUDA(holo_launch_kernel(ctx, dequant_activation_kernel, dim3((uint32_t)(want < cap ? want : cap)), dim3(256), 0, 1, in, out, n,
                                 (int)quant_dtype, (int)act, scale, (int)zero_point));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_reduce(holo_b200_ctx* ctx, const void* in, void* out, uint32_t rank, const uint32_t* dims, uint32_t axes_mask,
                           uint64_t n, int kind, int mean, uint8_t dtype) {
    ReduceParams p{};
    p.kind = kind, p.mean = mean, p.dtype = dtype;
    const bool full = rank == 0 || axes_mask == 0;
    uint64_t stride = 1;
    uint64_t strides[8];
    for (int i = (int)rank - 1; i >= 0; --i) {
        strides[i] = stride;
        stride *= dims[i];
    }
    p.out_count = 1, p.reduced_count = rank == 0 ? n : 1;
    for (uint32_t i = 0; i < rank; ++i) {
        if (full || ((axes_mask >> i) & 1u)) {
            p.red_dims[p.n_red] = dims[i], p.red_strides[p.n_red] = strides[i], ++p.n_red;
            p.reduced_count *= dims[i];
        } else {
            p.kept_dims[p.n_kept] = dims[i], p.kept_strides[p.n_kept] = strides[i], ++p.n_kept;
            p.out_count *= dims[i];
        }
    }
    if (rank == 0) p.red_dims[0] = (uint32_t)n, p.red_strides[0] = 1, p.n_red = 1;
    if (p.out_count == 1 && dtype == HOLO_DTYPE_F32 && kind != 1) {
        HOLO_CUDA(holo_launch_kernel(ctx, reduce_all_f32_kernel, dim3(1), dim3(1024), 0, 1, (const float*)in, (float*)out, n, kind, mean));
    } else {
        HOLO_CUDA(holo_launch_kernel(ctx, reduce_cells_kernel, dim3((uint32_t)((p.out_count + 127) / 128)), dim3(128), 0, 1, in, out, p));
    }
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_broadcast(holo_b200_ctx* ctx, const uint8_t* small, const uint8_t* other, uint8_t* out, uint32_t rank,
                              const uint32_t* in_dims, const uint32_t* out_dims, uint32_t es, int op, int small_is_lhs, uint8_t dtype) {
    BroadcastParams p{};
    p.rank = rank, p.es = es, p.op = op, p.small_is_lhs = small_is_lhs, p.dtype = dtype;
    uint64_t stride = 1, total = 1;
    for (int i = (int)rank - 1; i >= 0; --i) {
        p.out_dims[i] = out_dims[i];
        p.in_strides[i] = in_dims[i] == 1 ? 0 : stride;
        stride *= in_dims[i];
        total *= out_dims[i];
    }
    p.total = total;
    if (total == 0) return HOLO_OK;
    const uint64_t want = (total + 255) / 256, cap = (uint64_t)ctx->sm_count * 16;
    HOLO_CUDA(holo_launch_kernel(ctx, broadcast_kernel, dim3((uint32_t)(want < cap ? want : cap)), dim3(256), 0, 1, small, other, out, p));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_layer_norm(holo_b200_ctx* ctx, const void* x, const void* gamma, const void* beta, void* out, uint32_t batch,
                               uint32_t feature, float eps, uint8_t dtype) {
    if (batch == 0 || feature == 0) return HOLO_OK;
    const uint32_t threads = feature >= 1024 ? 256 : feature >= 128 ? 128 : 32;
    HOLO_CUDA(holo_launch_kernel(ctx, layer_norm_kernel, dim3(batch), dim3(threads), 0, 1, x, gamma, beta, out, feature, eps, (int)dtype));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_softmax(holo_b200_ctx* ctx, const void* x, void* out, uint32_t batch, uint32_t feature, uint8_t dtype) {
    if (batch == 0 || feature == 0) return HOLO_OK;
    const uint32_t threads = feature >= 1024 ? 256 : feature >= 128 ? 128 : 32;
    HOLO_CUDA(holo_launch_kernel(ctx, softmax_kernel, dim3(batch), dim3(threads), 0, 1, x, out, feature, (int)dtype));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_transpose(holo_b200_ctx* ctx, const uint8_t* in, uint8_t* out, uint32_t rank, const uint32_t* dims,
                              const uint8_t* perm, uint32_t es) {
    TransposeParams p = {};
    uint64_t in_strides[8], stride = 1;
    for (int i = (int)rank - 1; i >= 0; --i) {
        in_strides[i] = stride;
        stride *= dims[i];
    }
    p.total = stride;
    p.rank = rank;
    p.es = es;
    for (uint32_t i = 0; i < rank; ++i) {
        p.out_dims[i] = dims[perm[i]];
        p.in_strides_perm[i] = in_strides[perm[i]];
    }
    if (p.total == 0) return HOLO_OK;
    HOLO_CUDA(holo_launch_kernel(ctx, transpose_kernel, dim3(ew_blocks(p.total)), dim3(EW_THREADS), 0, 1, in, out, p));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_rope(holo_b200_ctx* ctx, const void* x, const void* c, const void* s, void* out, uint32_t head_dim,
                         uint64_t n, uint8_t dtype) {
    if (n == 0) return HOLO_OK;
    if (ctx->record) {
        HoloMicroOp m = {};
        m.kind = HOLO_MICRO_ROPE;
        m.p0 = x; m.p1 = c; m.p2 = s; m.o0 = out; m.a = head_dim; m.n = n; m.dtype = dtype;
        record_op(ctx, m, ew_blocks(n));
        return HOLO_OK;
    }
    HOLO_CUDA(holo_launch_kernel(ctx, rope_kernel, dim3(ew_blocks(n)), dim3(EW_THREADS), 0, 1, x, c, s, out, head_dim, n, dtype));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_gather(holo_b200_ctx* ctx, const uint8_t* data, const void* idx, uint8_t idx_dtype, uint8_t* out,
                           uint64_t outer, uint64_t axis_dim, uint64_t inner_bytes, uint64_t num_idx) {
    if (outer == 0 || num_idx == 0 || inner_bytes == 0) return HOLO_OK;
    if (outer > 65535) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "gather: outer %llu exceeds 65535", (unsigned long long)outer);
    dim3 grid((unsigned)num_idx, (unsigned)outer);
    HOLO_CUDA(holo_launch_kernel(ctx, gather_kernel, dim3(grid), dim3(128), 0, 1, data, idx, idx_dtype, out, axis_dim, inner_bytes, num_idx, ctx->dev_status));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_cast(holo_b200_ctx* ctx, const void* in, uint8_t src, void* out, uint8_t dst, uint64_t n) {
    if (n == 0) return HOLO_OK;
    HOLO_CUDA(holo_launch_kernel(ctx, cast_kernel, dim3(ew_blocks(n)), dim3(EW_THREADS), 0, 1, in, src, out, dst, n));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_dequantize(holo_b200_ctx* ctx, const HoloDequantizeCall& c, const void* in, const float* scales,
                               const int32_t* zps, void* out) {
    if (c.element_count == 0) return HOLO_OK;
    float scale;
    uint32_t sb = c.scale_bits;
    memcpy(&scale, &sb, 4);
    HOLO_CUDA(holo_launch_kernel(ctx, dequantize_kernel, dim3(ew_blocks(c.element_count)), dim3(EW_THREADS), 0, 1, 
        in, c.quant_dtype, scales, zps, c.channels, c.inner ? c.inner : 1, scale, c.zero_point, out, c.dtype,
        c.element_count));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_kv_write(holo_b200_ctx* ctx, const uint8_t* cache, const uint8_t* newr, const uint32_t* pos,
                             uint8_t* out, uint32_t planes, uint32_t bucket, uint32_t new_rows, uint32_t row_bytes) {
    if (planes == 0) return HOLO_OK;
    if (ctx->record) {
        if (out != cache || new_rows == 0) {   // only the in-place form is a pure row scatter
            ctx->record_failed = true;
            return HOLO_OK;
        }
        HoloMicroOp m = {};
        m.kind = HOLO_MICRO_KV_WRITE;
        m.p0 = newr; m.p1 = pos; m.o0 = out; m.a = planes; m.b = bucket; m.c = new_rows; m.d = row_bytes;
        record_op(ctx, m, ((uint64_t)planes * new_rows + 7) / 8);
        return HOLO_OK;
    }
    if (out != cache)
        HOLO_CUDA(cudaMemcpyAsync(out, cache, (size_t)planes * bucket * row_bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    if (new_rows == 0) return HOLO_OK;
    if (planes > 65535) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "kv_cache_write: planes %u exceeds 65535", planes);
    dim3 grid(new_rows, planes);
    HOLO_CUDA(holo_launch_kernel(ctx, kv_write_rows_kernel, dim3(grid), dim3(32), 0, 1, newr, pos, out, bucket, new_rows, row_bytes));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_rope_quantize(holo_b200_ctx* ctx, const void* x, const void* c, const void* s, void* rope_out, int8_t* codes,
                                  float* scales, uint64_t rows, uint32_t d, uint8_t dtype) {
    if (rows == 0 || d == 0) return HOLO_OK;
    const int warps = 8;
    const uint64_t blocks = (rows + warps - 1) / warps;
    if (blocks > 0x7fffffffull) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "rope_quantize_rows_i8: too many rows");
    if (ctx->record) {
        HoloMicroOp m = {};
        m.kind = HOLO_MICRO_ROPE_QUANT;
        m.p0 = x; m.p1 = c; m.p2 = s; m.o0 = rope_out; m.o1 = codes; m.o2 = scales; m.a = d; m.n = rows; m.dtype = dtype;
        record_op(ctx, m, blocks);
        return HOLO_OK;
    }
    HOLO_CUDA(holo_launch_kernel(ctx, rope_quantize_kernel, dim3((unsigned)blocks), dim3(warps * 32), 0, 1, x, c, s, rope_out, codes, scales, rows,
                                 d, (int)dtype));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}

int32_t holo_launch_quantize_rows(holo_b200_ctx* ctx, const void* x, uint8_t dtype, uint64_t rows, uint32_t d,
                                  int8_t* codes, float* scales) {
    if (rows == 0 || d == 0) return HOLO_OK;
    const int warps = 8;
    uint64_t blocks = (rows + warps - 1) / warps;
    if (blocks > 0x7fffffffull) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "quantize_rows_i8: too many rows");
    const bool vec = dtype != HOLO_DTYPE_F32 && (d % 128) == 0 && (((uintptr_t)x & 7u) == 0) && (((uintptr_t)codes & 3u) == 0);
    if (ctx->record) {
        HoloMicroOp m = {};
        m.kind = vec ? HOLO_MICRO_QUANT_VEC : HOLO_MICRO_QUANT;
        m.p0 = x; m.o0 = codes; m.o1 = scales; m.a = d; m.n = rows; m.dtype = dtype;
        record_op(ctx, m, blocks);
        return HOLO_OK;
    }
    if (vec)
        HOLO_CUDA(holo_launch_kernel(ctx, quantize_rows16_vec_kernel, dim3((unsigned)blocks), dim3(warps * 32), 0, 1, (const uint16_t*)x, dtype, rows, d, codes, scales));
    else
        HOLO_CUDA(holo_launch_kernel(ctx, quantize_rows_kernel, dim3((unsigned)blocks), dim3(warps * 32), 0, 1, x, dtype, rows, d, codes, scales));
    LAUNCH_CHECK(ctx);
    return HOLO_OK;
}
