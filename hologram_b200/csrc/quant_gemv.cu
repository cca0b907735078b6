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

    // ---- columns: one warp per column, grid-stride ----
    const uint32_t nvec = k >> 4;   // whole 16-byte pieces of a column's k-vector
    for (uint32_t col = blockIdx.x * QG_WARPS + warp; col < n; col += gridDim.x * QG_WARPS) {
        if (lane == 0 && zero_points && zero_points[col] != 0) atomicOr(status, 16u);   // the W8A8 form is symmetric
        const int8_t* w = bq + (uint64_t)col * k;
        int acc[QG_MAX_ROWS];
#pragma unroll
        for (int r = 0; r < QG_MAX_ROWS; ++r) acc[r] = 0;
        const bool vec_ok = ((uintptr_t)w & 15u) == 0;
        if (vec_ok) {
            for (uint32_t v = lane; v < nvec; v += 32) {
                const int4 wv = __ldg(reinterpret_cast<const int4*>(w) + v);
#pragma unroll
                for (int r = 0; r < QG_MAX_ROWS; ++r) {
                    if ((uint32_t)r < rows) {
                        const int4 qv = *reinterpret_cast<const int4*>(s_q + (size_t)r * kpad + (size_t)v * 16);
                        acc[r] = __dp4a(wv.x, qv.x, acc[r]);
                        acc[r] = __dp4a(wv.y, qv.y, acc[r]);
                        acc[r] = __dp4a(wv.z, qv.z, acc[r]);
                        acc[r] = __dp4a(wv.w, qv.w, acc[r]);
                    }
                }
            }
        }
        for (uint32_t j = (vec_ok ? nvec * 16 : 0) + lane; j < k; j += 32) {   // tail, or the whole column when unaligned
            const int wj = (int)w[j];
#pragma unroll
            for (int r = 0; r < QG_MAX_ROWS; ++r)
                if ((uint32_t)r < rows) acc[r] += wj * (int)s_q[(size_t)r * kpad + j];
        }
#pragma unroll
        for (int r = 0; r < QG_MAX_ROWS; ++r) {
            if ((uint32_t)r >= rows) break;
            int s = acc[r];
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);   // integer: any order is exact
            if (lane == 0) {
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
    const uint32_t want = (n + QG_WARPS - 1) / QG_WARPS, cap = 4u * (uint32_t)ctx->sm_count;
    const uint32_t grid = want < cap ? want : cap;
    for (uint32_t m0 = 0; m0 < m; m0 += per) {
        const uint32_t take = m - m0 < per ? m - m0 : per;
        HOLO_CUDA(holo_launch_kernel(ctx, matmul_w8a8_omajor_kernel, dim3(grid), dim3(QG_WARPS * 32), (size_t)take * kpad, 1, a, bq, scales,
                                     zero_points, residual, out, m0, take, k, n, act, ctx->dev_status));
        ctx->launches++;
    }
    return HOLO_OK;
}
