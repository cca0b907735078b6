// Output-major W8A8 decode product: out[m, n] = A[m, k] . dequant(Bq)^T for a symmetric per-channel
// int8 weight stored [n, k] (each output's k-vector contiguous), with per-token dynamic activation
// quantization. Replaces matmul_i8_pc_omajor (crates/hologram-compute/src/cpu/simd.rs:5278-5420,
// reached from matmul_dequant_float, cpu/float_kernels.rs:534-596) and its fused epilogue
// (matmul_dequant_epilogue, :727-766).
//
// Exact-integer contract: every activation row is quantized with quantize_row_i8
// (cpu/simd.rs:4761-4785: amax, inv = 127/amax, round half away from zero, clamp +-127,
// scale_a = amax/127), the dot is an exact i32 sum, and one f32 writeback
// (acc as f32) * (scale_a * scales[j]) follows: bit-identical to the CPU kernel whatever the
// order of the sum. A zero row gives a zero output row.
//
// HBM-bound on the weight (n*k bytes): one warp per output column at a time, lanes striding
// the column's k-vector with 128-bit loads and four dp4a per 16 bytes and activation row; the
// activation rows are quantized once per CTA into shared memory. Up to 8 rows per pass.
#include "common.h"
#include "numerics.cuh"

namespace {

constexpr int QG_WARPS = 8;
constexpr int QG_MAX_ROWS = 8;
constexpr int QG_UNROLL = 8;

// streaming weight load: read once, keep it out of L1
__device__ __forceinline__ int4 ld_weight(const int4* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__global__ void __launch_bounds__(QG_WARPS * 32)
matmul_w8a8_omajor_kernel(const float* __restrict__ a, const int8_t* __restrict__ bq, const float* __restrict__ scales,
                          const int32_t* __restrict__ zero_points, const float* __restrict__ residual, float* __restrict__ out,
                          uint32_t m0, uint32_t rows, uint32_t k, uint32_t n, int act, uint32_t* status) {
    holo_pdl_trigger();
    holo_pdl_wait();
    extern __shared__ __align__(16) int8_t s_q[];          // [rows][kpad] quantized activations
    __shared__ float s_scale[QG_MAX_ROWS];
    __shared__ float s_red[QG_WARPS];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t kpad = (k + 15u) & ~15u;

    const uint32_t nvec = k >> 4;   // whole 16-byte pieces of a column's k-vector
    const uint32_t nwarps = gridDim.x * QG_WARPS;
    const bool vec_ok = ((uintptr_t)bq & 15u) == 0 && (k & 15u) == 0;   // every column starts on a 16-byte boundary
    // The first weight batch of this warp's first two columns is requested before the activation
    // rows are quantized, so the weight stream is already running while the CTA does that.
    int4 wa[QG_UNROLL], wb[QG_UNROLL];
    const uint32_t first_col = blockIdx.x * QG_WARPS + warp;
    bool prefetched = false;
    if (vec_ok && first_col < n) {
        const bool two = first_col + nwarps < n;
        const int4* w0 = reinterpret_cast<const int4*>(bq + (uint64_t)first_col * k);
        const int4* w1 = reinterpret_cast<const int4*>(bq + (uint64_t)(two ? first_col + nwarps : first_col) * k);
#pragma unroll
        for (int u = 0; u < QG_UNROLL; ++u) {
            const uint32_t v = lane + 32 * u;
            wa[u] = make_int4(0, 0, 0, 0);
            wb[u] = make_int4(0, 0, 0, 0);
            if (v < nvec) {
                wa[u] = ld_weight(w0 + v);
                if (two) wb[u] = ld_weight(w1 + v);
            }
        }
        prefetched = true;
    }

    // ---- quantize_row_i8 of each activation row (every CTA does all rows: they are tiny) ----
    for (uint32_t r = 0; r < rows; ++r) {
        const float* row = a + (uint64_t)(m0 + r) * k;
        float amax = 0.0f;
        for (uint32_t j = tid; j < k; j += blockDim.x) {
            const float v = row[j], av = v < 0.0f ? -v : v;
            if (av > amax) amax = av;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, amax, o);
            if (other > amax) amax = other;
        }
        if (lane == 0) s_red[warp] = amax;
        __syncthreads();
        amax = s_red[0];
        for (int w = 1; w < QG_WARPS; ++w)
            if (s_red[w] > amax) amax = s_red[w];
        const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(127.0f, amax);
        for (uint32_t j = tid; j < kpad; j += blockDim.x) {
            int q = 0;
            if (j < k && amax != 0.0f) {
                const float t = __fmul_rn(row[j], inv);
                q = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
                q = max(-127, min(127, q));
            }
            s_q[(size_t)r * kpad + j] = (int8_t)q;
        }
        if (tid == 0) s_scale[r] = amax == 0.0f ? 0.0f : __fdiv_rn(amax, 127.0f);
        __syncthreads();
    }

    // ---- columns: each warp takes two columns at a time (grid-stride), four 128-bit weight loads
    // per lane and column in flight before the first dp4a ----
    for (uint32_t col0 = first_col; col0 < n; col0 += 2 * nwarps) {
        const uint32_t col1 = col0 + nwarps;
        const bool two = col1 < n;
        if (lane == 0 && zero_points && (zero_points[col0] != 0 || (two && zero_points[col1] != 0))) atomicOr(status, 16u);   // symmetric form only
        const int8_t* w0 = bq + (uint64_t)col0 * k;
        const int8_t* w1 = bq + (uint64_t)(two ? col1 : col0) * k;
        int acc0[QG_MAX_ROWS], acc1[QG_MAX_ROWS];
#pragma unroll
        for (int r = 0; r < QG_MAX_ROWS; ++r) acc0[r] = acc1[r] = 0;
        if (vec_ok) {
            for (uint32_t v0 = lane; v0 < nvec; v0 += 32 * QG_UNROLL) {
                if (!(prefetched && v0 == lane)) {
#pragma unroll
                    for (int u = 0; u < QG_UNROLL; ++u) {
                        const uint32_t v = v0 + 32 * u;
                        wa[u] = make_int4(0, 0, 0, 0);
                        wb[u] = make_int4(0, 0, 0, 0);
                        if (v < nvec) {
                            wa[u] = ld_weight(reinterpret_cast<const int4*>(w0) + v);
                            if (two) wb[u] = ld_weight(reinterpret_cast<const int4*>(w1) + v);
                        }
                    }
                }
                prefetched = false;
#pragma unroll
                for (int u = 0; u < QG_UNROLL; ++u) {
                    const uint32_t v = v0 + 32 * u;
                    if (v >= nvec) continue;
#pragma unroll
                    for (int r = 0; r < QG_MAX_ROWS; ++r) {
                        if ((uint32_t)r < rows) {
                            const int4 qv = *reinterpret_cast<const int4*>(s_q + (size_t)r * kpad + (size_t)v * 16);
                            acc0[r] = __dp4a(wa[u].x, qv.x, acc0[r]);
                            acc0[r] = __dp4a(wa[u].y, qv.y, acc0[r]);
                            acc0[r] = __dp4a(wa[u].z, qv.z, acc0[r]);
                            acc0[r] = __dp4a(wa[u].w, qv.w, acc0[r]);
                            acc1[r] = __dp4a(wb[u].x, qv.x, acc1[r]);
                            acc1[r] = __dp4a(wb[u].y, qv.y, acc1[r]);
                            acc1[r] = __dp4a(wb[u].z, qv.z, acc1[r]);
                            acc1[r] = __dp4a(wb[u].w, qv.w, acc1[r]);
                        }
                    }
                }
            }
        } else {
            for (uint32_t j = lane; j < k; j += 32) {
                const int a0 = (int)w0[j], a1 = two ? (int)w1[j] : 0;
#pragma unroll
                for (int r = 0; r < QG_MAX_ROWS; ++r)
                    if ((uint32_t)r < rows) {
                        const int q = (int)s_q[(size_t)r * kpad + j];
                        acc0[r] += a0 * q;
                        acc1[r] += a1 * q;
                    }
            }
        }
#pragma unroll
        for (int r = 0; r < QG_MAX_ROWS; ++r) {
            if ((uint32_t)r >= rows) break;
            int s0 = acc0[r], s1 = acc1[r];
            for (int o = 16; o > 0; o >>= 1) {   // integer: any order is exact
                s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                s1 += __shfl_xor_sync(0xffffffffu, s1, o);
            }
            if (lane < 2 && (lane == 0 || two)) {
                const uint32_t col = lane == 0 ? col0 : col1;
                const int s = lane == 0 ? s0 : s1;
                const float sa = s_scale[r];
                const uint64_t idx = (uint64_t)(m0 + r) * n + col;
                float y = sa == 0.0f ? 0.0f : __fmul_rn(__int2float_rn(s), __fmul_rn(sa, scales[col]));
                if (residual) y = __fadd_rn(y, residual[idx]);
                if (act >= 0) y = holo::lut_act_ref(act, y);
                out[idx] = y;
            }
        }
    }
}

}  // namespace

int32_t holo_launch_matmul_w8a8_omajor(holo_b200_ctx* ctx, const float* a, const int8_t* bq, const float* scales, const int32_t* zero_points,
                                       const float* residual, float* out, uint32_t m, uint32_t k, uint32_t n, int act) {
    if (m == 0 || k == 0 || n == 0) return HOLO_OK;
    const uint32_t kpad = (k + 15u) & ~15u;
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        HOLO_CUDA(cudaFuncSetAttribute(matmul_w8a8_omajor_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured_device = ctx->device;
    }
    uint32_t per = QG_MAX_ROWS;   // rows per launch: what fits the shared-memory activation buffer
    while (per > 1 && (size_t)per * kpad > 200 * 1024) per >>= 1;
    if ((size_t)per * kpad > 200 * 1024)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: k %u does not fit the shared-memory activation row", k);
    const uint32_t want = (n + 2 * QG_WARPS - 1) / (2 * QG_WARPS), cap = 2u * (uint32_t)ctx->sm_count;   // persistent: every CTA quantizes the rows once
    const uint32_t grid = want < cap ? want : cap;
    for (uint32_t m0 = 0; m0 < m; m0 += per) {
        const uint32_t take = m - m0 < per ? m - m0 : per;
        HOLO_CUDA(holo_launch_kernel(ctx, matmul_w8a8_omajor_kernel, dim3(grid), dim3(QG_WARPS * 32), (size_t)take * kpad, 1, a, bq, scales,
                                     zero_points, residual, out, m0, take, k, n, act, ctx->dev_status));
        ctx->launches++;
    }
    return HOLO_OK;
}
