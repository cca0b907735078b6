// General-shape decode attention (any head_dim, any GQA group, any q_rows, f32/f16/bf16 or
// int8-coded K/V). One CTA per output row; its warps take interleaved keys with a running
// (max, sum, context) triple each and merge through shared memory at the end. Used for the
// shapes the tiled tensor-core kernel does not cover.
// Follows decode_attention_valid_row (crates/hologram-compute/src/cpu/float_kernels.rs:3834-3883):
// score = dot(q, k) / scale; softmax over the visible keys; context = sum p * v.
#pragma once
#include "common.h"
#include "numerics.cuh"

namespace holo_attn {

constexpr int GEN_WARPS = 8;
constexpr int GEN_MAX_PER_LANE = 16;  // head_dim <= 512

template <bool Q8>
__device__ __forceinline__ float kv_elem(const void* base, const float* scales, uint64_t row, uint32_t d, uint32_t c,
                                         int dtype) {
    if (Q8) {
        // Dequantize with zero-point 0 (cpu/kernels.rs:262): (q as f32) * scale
        return __fmul_rn(__int2float_rn((int)((const int8_t*)base)[row * d + c]), scales[row]);
    } else {
        return holo::load_float(base, row * d + c, dtype);
    }
}

template <bool Q8>
__global__ void __launch_bounds__(GEN_WARPS * 32)
decode_attention_generic_kernel(HoloAttnArgs a) {
    holo_pdl_trigger();
    holo_pdl_wait();
    extern __shared__ float s_mem[];  // [GEN_WARPS][d + 2]
    const uint32_t r = blockIdx.x;    // output row: (batch, head, query row)
    const uint32_t d = a.d, h = a.h, m = a.m, hkv = a.hkv;
    const uint32_t bi = r / (h * m), hi = (r / m) % h, qi = r % m;
    const uint32_t kvh = bi * hkv + hi / (h / hkv);
    // scalar-mask form: the first min(valid_len, past) cache rows, then chunk rows 0..qi;
    // additive-mask form (decode_attention_row, cpu/float_kernels.rs:2420-2477): every key, the
    // mask row added to the scaled score
    const uint32_t vis_past = a.mask || !a.valid_len ? a.past : min(*a.valid_len, a.past);
    const uint32_t new_vis = a.mask || a.all_new ? a.nnew : min(qi + 1, a.nnew);
    const float* mask_row = a.mask ? a.mask + (uint64_t)qi * (a.past + a.nnew) : nullptr;
    const uint32_t vis = vis_past + new_vis;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    float q[GEN_MAX_PER_LANE], o[GEN_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < GEN_MAX_PER_LANE; ++i) {
        uint32_t c = lane + 32 * i;
        q[i] = c < d ? holo::load_float(a.q, (uint64_t)r * d + c, a.dtype) : 0.0f;
        o[i] = 0.0f;
    }
    float mx = -INFINITY, sum = 0.0f;
    for (uint32_t kj = warp; kj < vis; kj += GEN_WARPS) {
        const bool past = kj < vis_past;
        const void* kb = past ? a.k_past : a.k_new;
        const void* vb = past ? a.v_past : a.v_new;
        const float* ks = past ? a.k_past_s : a.k_new_s;
        const float* vs = past ? a.v_past_s : a.v_new_s;
        const uint64_t row = past ? (uint64_t)kvh * a.past + kj : (uint64_t)kvh * a.nnew + (kj - vis_past);
        float part = 0.0f;
#pragma unroll
        for (int i = 0; i < GEN_MAX_PER_LANE; ++i) {
            uint32_t c = lane + 32 * i;
            if (c < d) part = fmaf(q[i], kv_elem<Q8>(kb, ks, row, d, c, a.dtype), part);
        }
        for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        float s = __fdiv_rn(part, a.scale_div);
        if (mask_row) {
            s = __fadd_rn(s, mask_row[kj]);
            if (s == -INFINITY) continue;   // erased exactly: contributes 0 to the sum and the context
        }
        const float nm = fmaxf(mx, s);
        const float corr = mx == -INFINITY ? 0.0f : expf(mx - nm);
        const float p = expf(s - nm);
        sum = sum * corr + p;
#pragma unroll
        for (int i = 0; i < GEN_MAX_PER_LANE; ++i) {
            uint32_t c = lane + 32 * i;
            if (c < d) o[i] = fmaf(p, kv_elem<Q8>(vb, vs, row, d, c, a.dtype), o[i] * corr);
        }
        mx = nm;
    }
    float* mine = s_mem + (size_t)warp * (d + 2);
#pragma unroll
    for (int i = 0; i < GEN_MAX_PER_LANE; ++i) {
        uint32_t c = lane + 32 * i;
        if (c < d) mine[c] = o[i];
    }
    if (lane == 0) {
        mine[d] = mx;
        mine[d + 1] = sum;
    }
    __syncthreads();
    float gm = -INFINITY;
    for (int w = 0; w < GEN_WARPS; ++w) gm = fmaxf(gm, s_mem[(size_t)w * (d + 2) + d]);
    float gs = 0.0f;
    for (int w = 0; w < GEN_WARPS; ++w) {
        float wm = s_mem[(size_t)w * (d + 2) + d];
        if (wm != -INFINITY) gs += s_mem[(size_t)w * (d + 2) + d + 1] * expf(wm - gm);
    }
    const float denom = fmaxf(gs, 1e-30f);
    for (uint32_t c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.0f;
        for (int w = 0; w < GEN_WARPS; ++w) {
            float wm = s_mem[(size_t)w * (d + 2) + d];
            if (wm != -INFINITY) acc += s_mem[(size_t)w * (d + 2) + c] * expf(wm - gm);
        }
        // zero visible keys (or every key erased by the mask) => exact zero vector
        // (cpu/float_kernels.rs:3851-3854, 2451-2454)
        holo::store_float(a.out, (uint64_t)r * d + c, (vis == 0 || gm == -INFINITY) ? 0.0f : acc / denom, a.dtype);
    }
}

}  // namespace holo_attn
