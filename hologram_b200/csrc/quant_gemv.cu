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

// quantize_row_i8 (cpu/simd.rs:4761-4785) of `rows` activation rows into shared memory [rows][kpad]; every
// thread of the CTA takes part (QG_WARPS warps), and every CTA does all rows: they are tiny.
// `chunk` != 0 (E8 tier): the 8-element groups of a row are stored transposed in blocks of 16, group g at
// position (g % 16) * chunk + g / 16 (chunk = groups / 16), so that lanes holding sixteen consecutive indices each
// read neighbouring 8-byte groups at every step instead of the same bank.
__device__ __forceinline__ void quantize_rows_to_shared(const float* __restrict__ a, uint32_t m0, uint32_t rows, uint32_t k, uint32_t kpad,
                                                        int8_t* s_q, float* s_scale, float* s_red, uint32_t chunk = 0) {
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
            const uint32_t g = j >> 3;
            const uint32_t pos = chunk ? ((g & 15u) * chunk + (g >> 4)) * 8 + (j & 7u) : j;
            s_q[(size_t)r * kpad + pos] = (int8_t)q;
        }
        if (tid == 0) s_scale[r] = amax == 0.0f ? 0.0f : __fdiv_rn(amax, 127.0f);
        __syncthreads();
    }

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

    quantize_rows_to_shared(a, m0, rows, k, kpad, s_q, s_scale, s_red);

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

// E8 codebook tier (W1A8; matmul_e8cb_omajor, cpu/simd.rs:6845-6960): the weight is [n, k/8] bytes, each the index of
// an 8-element i8 block of the model's 256 x 8 codebook (a constant operand); otherwise the i8 product: quantized
// row, exact i32 dot, one f32 writeback. The index stream is an eighth of the i8 weight, so the kernel is bound by
// the dp4a count and the shared-memory lookups, not by HBM: the codebook (2 KiB) and the rows sit in shared memory,
// one warp per column, a lane takes sixteen indices per 128-bit load.
__global__ void __launch_bounds__(QG_WARPS * 32)
matmul_e8cb_omajor_kernel(const float* __restrict__ a, const uint8_t* __restrict__ bq, const int8_t* __restrict__ codebook,
                          const float* __restrict__ scales, const int32_t* __restrict__ zero_points, const float* __restrict__ residual,
                          float* __restrict__ out, uint32_t m0, uint32_t rows, uint32_t k, uint32_t n, int act, uint32_t* status) {
    holo_pdl_trigger();
    holo_pdl_wait();
    extern __shared__ __align__(16) int8_t s_q[];          // [rows][kpad] quantized activations
    __shared__ __align__(16) int2 s_cb[256];
    __shared__ float s_scale[QG_MAX_ROWS];
    __shared__ float s_red[QG_WARPS];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t kpad = (k + 15u) & ~15u, groups = k >> 3;
    for (uint32_t i = tid; i < 256; i += blockDim.x) {
        const int8_t* e = codebook + (size_t)i * 8;
        s_cb[i] = make_int2((int)((uint32_t)(uint8_t)e[0] | ((uint32_t)(uint8_t)e[1] << 8) | ((uint32_t)(uint8_t)e[2] << 16) | ((uint32_t)(uint8_t)e[3] << 24)),
                            (int)((uint32_t)(uint8_t)e[4] | ((uint32_t)(uint8_t)e[5] << 8) | ((uint32_t)(uint8_t)e[6] << 16) | ((uint32_t)(uint8_t)e[7] << 24)));
    }
    const bool vec_ok = ((uintptr_t)bq & 15u) == 0 && (groups & 15u) == 0;   // every column's indices start on a 16-byte boundary
    const uint32_t chunk = vec_ok ? groups >> 4 : 0;
    quantize_rows_to_shared(a, m0, rows, k, kpad, s_q, s_scale, s_red, chunk);   // ends with a barrier: the codebook is in place too

    for (uint32_t col = blockIdx.x * QG_WARPS + warp; col < n; col += gridDim.x * QG_WARPS) {
        if (lane == 0 && zero_points && zero_points[col] != 0) atomicOr(status, 16u);   // symmetric form only
        const uint8_t* idx = bq + (uint64_t)col * groups;
        int acc[QG_MAX_ROWS];
#pragma unroll
        for (int r = 0; r < QG_MAX_ROWS; ++r) acc[r] = 0;
        auto group = [&](uint32_t g, uint32_t code) {
            const int2 w = s_cb[code];
#pragma unroll
            for (int r = 0; r < QG_MAX_ROWS; ++r)
                if ((uint32_t)r < rows) {
                    const int2 q = *reinterpret_cast<const int2*>(s_q + (size_t)r * kpad + (size_t)g * 8);   // g = the group's position in the row
                    acc[r] = __dp4a(w.x, q.x, acc[r]);
                    acc[r] = __dp4a(w.y, q.y, acc[r]);
                }
        };
        if (vec_ok) {
            for (uint32_t v = lane; v < (groups >> 4); v += 32) {
                const int4 w = ld_weight(reinterpret_cast<const int4*>(idx) + v);
                const uint32_t words[4] = {(uint32_t)w.x, (uint32_t)w.y, (uint32_t)w.z, (uint32_t)w.w};
#pragma unroll
                for (int j = 0; j < 16; ++j) group(j * chunk + v, (words[j >> 2] >> (8 * (j & 3))) & 255u);   // index 16 v + j, stored at j * chunk + v
            }
        } else {
            for (uint32_t g = lane; g < groups; g += 32) group(g, idx[g]);
        }
#pragma unroll
        for (int r = 0; r < QG_MAX_ROWS; ++r) {
            if ((uint32_t)r >= rows) break;
            int sum = acc[r];
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);   // integer: any order is exact
            if (lane == 0) {
                const float sa = s_scale[r];
                const uint64_t o = (uint64_t)(m0 + r) * n + col;
                float y = sa == 0.0f ? 0.0f : __fmul_rn(__int2float_rn(sum), __fmul_rn(sa, scales[col]));
                if (residual) y = __fadd_rn(y, residual[o]);
                if (act >= 0) y = holo::lut_act_ref(act, y);
                out[o] = y;
            }
        }
    }
}

// ---- stream form: the weight is one contiguous [n, k] byte stream, so it is brought in like any
// other stream: a copy warp keeps a ring of bulk async copies in flight (tiles of whole columns)
// and the bytes in flight do not depend on registers. The eight product warps form four groups of
// two that take tiles in turn (so one group's reduction and write-back overlap the others'
// products); inside a group the warps split the tile's k range. Taken when k is a multiple of 16,
// at most QS_STAGE_BYTES, and the weight is 16-byte aligned.
// Measured on B200: dp4a issues at about 16 lanes per clock per SM, so from four activation rows on
// the product is bound by dp4a, not by HBM; the same loop on mma.sync.m16n8k32.s8 (weights as the B
// operand) was slower at every row count.
constexpr int QS_GROUPS = 4;
constexpr int QS_GROUP_WARPS = 2;
constexpr int QS_WARPS = QS_GROUPS * QS_GROUP_WARPS;   // product warps; warp QS_WARPS is the copy warp
constexpr int QS_MAX_STAGES = 12;             // as many as fit beside the quantized rows: the ring must cover DRAM latency plus the tiles being consumed
constexpr int QS_MIN_STAGES = 5;
constexpr uint32_t QS_STAGE_BYTES = 16384;
constexpr int QS_MAX_COLS = 4;                 // columns per tile (8 for the packed-i4 weight up to four rows: its columns are half as long)
__host__ __device__ constexpr int qs_max_cols(int rows, bool i4) { return i4 && rows <= 4 ? 2 * QS_MAX_COLS : QS_MAX_COLS; }
constexpr uint32_t QS_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t qs_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool qs_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    for (uint32_t it = 0; it < QS_WAIT_LIMIT && !ok; ++it) {
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    }
    return ok != 0;
}
__device__ __forceinline__ void qs_product_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(QS_WARPS * 32) : "memory"); }
__device__ __forceinline__ void qs_group_barrier(uint32_t group) {
    asm volatile("bar.sync %0, %1;" ::"r"(2 + group), "n"(QS_GROUP_WARPS * 32) : "memory");
}

// Sums V values over the 32 lanes with about V shuffles instead of 5 V: at each step a lane keeps
// one value of a pair and hands the other to its partner, so the number of live values halves.
// Afterwards the total of value index `idx` sits in the lanes whose bits 4, 3, ... spell idx
// (bit t of idx = lane bit 4 - t); exact for integers whatever the order.
template <int V>
__device__ __forceinline__ int qs_reduce(int (&vals)[V], uint32_t lane) {
    int live = V;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        if (live > 1) {
#pragma unroll
            for (int j = 0; j < V / 2; ++j) {
                if (j < live / 2) {
                    const int x = vals[2 * j], y = vals[2 * j + 1];
                    const bool hi = (lane & o) != 0;
                    vals[j] = (hi ? y : x) + __shfl_xor_sync(0xffffffffu, hi ? x : y, o);
                }
            }
            live >>= 1;
        } else {
            vals[0] += __shfl_xor_sync(0xffffffffu, vals[0], o);
        }
    }
    return vals[0];
}
template <int V>
__device__ __forceinline__ uint32_t qs_reduce_index(uint32_t lane) {
    uint32_t idx = 0;
#pragma unroll
    for (int t = 0; (1 << t) < V; ++t) idx |= ((lane >> (4 - t)) & 1u) << t;
    return idx;
}

// shared memory: [ROWS * k quantized rows][stages * QS_STAGE_BYTES ring][2 parities * QS_WARPS * 32 partial sums]
//                [QS_MAX_ROWS scales][QS_WARPS maxima][abort flag][QS_MAX_ROWS row sums][2 * QS_MAX_STAGES mbarriers]
__host__ __device__ constexpr size_t qs_smem_bytes(uint32_t rows, uint32_t k, uint32_t stages) {
    return (size_t)rows * k + (size_t)stages * QS_STAGE_BYTES + 2 * QS_WARPS * 32 * 4 + QG_MAX_ROWS * 4 + QS_WARPS * 4 + 16 + QG_MAX_ROWS * 4 + 16 * QS_MAX_STAGES;
}
constexpr size_t QS_SMEM_LIMIT = 226 * 1024;

// I4 (matmul_i4_pc_omajor, cpu/simd.rs:6164-6260): the weight is [n, k/2] bytes of packed signed nibbles, low
// nibble first. A 32-bit weight word holds eight elements; (w ^ 0x88888888) & 0x0F0F0F0F are the even elements
// plus 8 and the same of w >> 4 the odd ones, so the quantized row is kept with the even and the odd elements
// of every eight in two separate words (two dp4a per weight word) and 8 * sum(row) is taken off at the end.
template <int ROWS, bool I4>
__global__ void __launch_bounds__((QS_WARPS + 1) * 32, 1)
matmul_w8a8_stream_kernel(const float* __restrict__ a, const int8_t* __restrict__ bq, const float* __restrict__ scales,
                          const int32_t* __restrict__ zero_points, const float* __restrict__ residual, float* __restrict__ out,
                          uint32_t m0, uint32_t rows, uint32_t k, uint32_t n, uint32_t cols_per_tile, uint32_t stages, int act, uint32_t* status) {
    constexpr int MAXC = qs_max_cols(ROWS, I4);
    constexpr int V = MAXC * ROWS;             // sums per tile
    static_assert(V <= 32, "one partial slot per lane");
    extern __shared__ __align__(128) unsigned char qs_mem[];
    int8_t* s_q = reinterpret_cast<int8_t*>(qs_mem);
    unsigned char* ring = qs_mem + (size_t)ROWS * k;
    int* s_part = reinterpret_cast<int*>(ring + (size_t)stages * QS_STAGE_BYTES);
    float* s_scale = reinterpret_cast<float*>(s_part + 2 * QS_WARPS * 32);
    float* s_red = s_scale + QG_MAX_ROWS;
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(s_red + QS_WARPS);
    int* s_sum = reinterpret_cast<int*>(s_red + QS_WARPS + 4);
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_sum + QG_MAX_ROWS);
    const uint32_t bar_full = qs_smem(bars), bar_empty = qs_smem(bars + QS_MAX_STAGES);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t ntiles = (n + cols_per_tile - 1) / cols_per_tile;
    const uint32_t kw = I4 ? k >> 1 : k;   // bytes of one weight column

    holo_pdl_trigger();
    if (tid == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_full + 8 * s));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_empty + 8 * s), "r"(QS_GROUP_WARPS));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *s_abort = 0;
        for (int r = 0; r < QG_MAX_ROWS; ++r) s_sum[r] = 0;
    }
    __syncthreads();
    holo_pdl_wait();  // nothing above touches global memory

    if (warp == QS_WARPS) {   // copy warp: tiles blockIdx.x, + gridDim.x, ... through the ring
        if (lane != 0) return;
        uint32_t i = 0;
        for (uint32_t t = blockIdx.x; t < ntiles; t += gridDim.x, ++i) {
            const uint32_t s = i % stages, use = i / stages;
            if (use > 0 && (*s_abort || !qs_wait(bar_empty + 8 * s, (use - 1) & 1))) {
                *s_abort = 1;
                atomicOr(status, 2u);
                break;
            }
            const uint32_t c0 = t * cols_per_tile, cols = n - c0 < cols_per_tile ? n - c0 : cols_per_tile;
            const uint32_t bytes = cols * kw;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_full + 8 * s), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(qs_smem(ring + (size_t)s * QS_STAGE_BYTES)), "l"(bq + (uint64_t)c0 * kw), "r"(bytes), "r"(bar_full + 8 * s) : "memory");
        }
        return;
    }

    // The writer threads of a group (one per column and row of a tile) fetch the column's scale, zero
    // point and residual one tile ahead, so that no global-memory latency sits between two tiles.
    const uint32_t group = warp / QS_GROUP_WARPS, gwarp = warp % QS_GROUP_WARPS, gtid = tid % (QS_GROUP_WARPS * 32);
    const uint32_t wc = gtid / ROWS, wr = gtid % ROWS;      // this writer's column within the tile, and row
    const bool writer = gtid < (uint32_t)V && wr < rows;
    float sc_next = 0.0f, res_next = 0.0f;
    int zp_next = 0;
    auto fetch_epilogue = [&](uint32_t tile) {
        sc_next = 0.0f, res_next = 0.0f, zp_next = 0;
        const uint64_t col = (uint64_t)tile * cols_per_tile + wc;
        if (writer && tile < ntiles && wc < cols_per_tile && col < n) {
            sc_next = scales[col];
            if (zero_points) zp_next = zero_points[col];
            if (residual) res_next = residual[(uint64_t)(m0 + wr) * n + col];
        }
    };
    fetch_epilogue(blockIdx.x + group * gridDim.x);

    // ---- quantize_row_i8 of the activation rows, while the first tiles are on their way. The rows
    // are done side by side (8 / ROWS warps each), with 128-bit loads issued sixteen at a time: the row
    // comes from L2 and every dependent round trip would cost as much as streaming a few tiles. Each
    // CTA starts its sweep of the row at a different 128-byte line, so that the CTAs do not all ask
    // the same L2 lines at the same moment. ----
    {
        constexpr uint32_t WPR = QS_WARPS / ROWS, QT = WPR * 32, QB = 16;
        const uint32_t qrow = warp / WPR, qtid = (warp % WPR) * 32 + lane;
        const bool qlive = qrow < rows;
        const float* row = a + (uint64_t)(m0 + (qlive ? qrow : 0)) * k;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const bool a_vec = ((uintptr_t)a & 15u) == 0;   // k is a multiple of 16, so every row then starts on a 16-byte boundary
        const uint32_t nq = k >> 2;
        const uint32_t rot = (uint32_t)(((uint64_t)blockIdx.x * nq) / gridDim.x) & ~7u;
        auto at = [&](uint32_t e) { return e + rot < nq ? e + rot : e + rot - nq; };   // e < nq
        float amax = 0.0f;
        auto upd = [&](float v) {
            const float av = v < 0.0f ? -v : v;
            if (av > amax) amax = av;
        };
        auto upd4 = [&](const float4& v) { upd(v.x), upd(v.y), upd(v.z), upd(v.w); };
        float4 first[QB];   // the first batch stays in registers for the second pass
        if (qlive && a_vec) {
#pragma unroll
            for (uint32_t u = 0; u < QB; ++u) {
                const uint32_t j = qtid + u * QT;
                first[u] = j < nq ? row4[at(j)] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (uint32_t u = 0; u < QB; ++u) upd4(first[u]);
            for (uint32_t j0 = qtid + QB * QT; j0 < nq; j0 += QB * QT) {
                float4 v[QB];
#pragma unroll
                for (uint32_t u = 0; u < QB; ++u) v[u] = j0 + u * QT < nq ? row4[at(j0 + u * QT)] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (uint32_t u = 0; u < QB; ++u) upd4(v[u]);
            }
        } else if (qlive) {
            for (uint32_t j = qtid; j < k; j += QT) upd(row[j]);
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, amax, o);
            if (other > amax) amax = other;
        }
        if (lane == 0) s_red[warp] = amax;
        qs_product_barrier();
        amax = s_red[qrow * WPR];
#pragma unroll
        for (uint32_t w = 1; w < WPR; ++w)
            if (s_red[qrow * WPR + w] > amax) amax = s_red[qrow * WPR + w];
        const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(127.0f, amax);
        auto quant1 = [&](float x) {
            const float t = __fmul_rn(x, inv);
            const int q = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
            return (uint32_t)(max(-127, min(127, q)) & 0xff);
        };
        int qsum = 0;   // I4: the row's sum of codes
        // the four codes of elements 4j .. 4j+3 go to their place in the row: in order (i8), or the even ones
        // to the first and the odd ones to the second word of the eight elements they belong to (i4)
        auto put4 = [&](uint32_t j, const float4& v) {
            const uint32_t q0 = amax == 0.0f ? 0u : quant1(v.x), q1 = amax == 0.0f ? 0u : quant1(v.y);
            const uint32_t q2 = amax == 0.0f ? 0u : quant1(v.z), q3 = amax == 0.0f ? 0u : quant1(v.w);
            int8_t* base = s_q + (size_t)qrow * k;
            if (I4) {
                qsum += (int)(int8_t)q0 + (int)(int8_t)q1 + (int)(int8_t)q2 + (int)(int8_t)q3;
                uint16_t* half = reinterpret_cast<uint16_t*>(base + (size_t)(j >> 1) * 8 + (j & 1) * 2);
                half[0] = (uint16_t)(q0 | (q2 << 8));
                half[2] = (uint16_t)(q1 | (q3 << 8));
            } else {
                reinterpret_cast<uint32_t*>(base)[j] = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
            }
        };
        if (qlive && a_vec) {
#pragma unroll
            for (uint32_t u = 0; u < QB; ++u)
                if (qtid + u * QT < nq) put4(at(qtid + u * QT), first[u]);
            for (uint32_t j0 = qtid + QB * QT; j0 < nq; j0 += QB * QT) {
                float4 v[QB];
#pragma unroll
                for (uint32_t u = 0; u < QB; ++u) v[u] = j0 + u * QT < nq ? row4[at(j0 + u * QT)] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (uint32_t u = 0; u < QB; ++u)
                    if (j0 + u * QT < nq) put4(at(j0 + u * QT), v[u]);
            }
        } else if (qlive) {
            for (uint32_t j = qtid; j < k; j += QT) {
                const int q = amax == 0.0f ? 0 : (int)(int8_t)quant1(row[j]);
                qsum += q;
                s_q[(size_t)qrow * k + (I4 ? (j >> 3) * 8 + (j & 1) * 4 + ((j & 7) >> 1) : j)] = (int8_t)q;
            }
        }
        if (I4) {
            for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
            if (qlive && lane == 0) atomicAdd(s_sum + qrow, qsum);
        }
        if (qlive && qtid == 0) s_scale[qrow] = amax == 0.0f ? 0.0f : __fdiv_rn(amax, 127.0f);
        qs_product_barrier();
    }

    const uint32_t nvec = kw >> 4;   // 16-byte weight units of a column
    const uint32_t ridx = qs_reduce_index<V>(lane);
    const bool rlane = (lane & ((32u / (V < 32 ? V : 32)) - 1u)) == 0;   // one lane per value index stores the warp's sum
    for (uint32_t i = group; ; i += QS_GROUPS) {
        const uint32_t t = blockIdx.x + i * gridDim.x;
        if (t >= ntiles) break;
        const uint32_t s = i % stages, use = i / stages;
        const uint32_t c0 = t * cols_per_tile, cols = n - c0 < cols_per_tile ? n - c0 : cols_per_tile;
        const float sc = sc_next, res = res_next;
        const int zp = zp_next;
        fetch_epilogue(t + QS_GROUPS * gridDim.x);
        const bool ok = !*s_abort && qs_wait(bar_full + 8 * s, use & 1);
        if (!ok) {   // keep walking so that every warp of the group still meets the barrier below
            *s_abort = 1;
            atomicOr(status, 2u);
        }
        int acc[V];
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = 0;
        if (ok) {
            const int4* tile = reinterpret_cast<const int4*>(ring + (size_t)s * QS_STAGE_BYTES);
#pragma unroll 2
            for (uint32_t v = gwarp * 32 + lane; v < nvec; v += QS_GROUP_WARPS * 32) {
                if (I4) {
                    // one 16-byte weight unit = 32 elements = 32 bytes of the row: words (even, odd) x 4
                    int4 qa[ROWS], qb[ROWS];
#pragma unroll
                    for (int r = 0; r < ROWS; ++r) {
                        qa[r] = *reinterpret_cast<const int4*>(s_q + (size_t)r * k + (size_t)v * 32);
                        qb[r] = *reinterpret_cast<const int4*>(s_q + (size_t)r * k + (size_t)v * 32 + 16);
                    }
#pragma unroll
                    for (int c = 0; c < MAXC; ++c) {
                        if ((uint32_t)c < cols) {
                            const int4 w = tile[(size_t)c * nvec + v];
                            const uint32_t x0 = (uint32_t)w.x ^ 0x88888888u, x1 = (uint32_t)w.y ^ 0x88888888u;
                            const uint32_t x2 = (uint32_t)w.z ^ 0x88888888u, x3 = (uint32_t)w.w ^ 0x88888888u;
#pragma unroll
                            for (int r = 0; r < ROWS; ++r) {
                                int x = acc[c * ROWS + r];
                                x = __dp4a((int)(x0 & 0x0F0F0F0Fu), qa[r].x, x);
                                x = __dp4a((int)((x0 >> 4) & 0x0F0F0F0Fu), qa[r].y, x);
                                x = __dp4a((int)(x1 & 0x0F0F0F0Fu), qa[r].z, x);
                                x = __dp4a((int)((x1 >> 4) & 0x0F0F0F0Fu), qa[r].w, x);
                                x = __dp4a((int)(x2 & 0x0F0F0F0Fu), qb[r].x, x);
                                x = __dp4a((int)((x2 >> 4) & 0x0F0F0F0Fu), qb[r].y, x);
                                x = __dp4a((int)(x3 & 0x0F0F0F0Fu), qb[r].z, x);
                                x = __dp4a((int)((x3 >> 4) & 0x0F0F0F0Fu), qb[r].w, x);
                                acc[c * ROWS + r] = x;
                            }
                        }
                    }
                    continue;
                }
                int4 qv[ROWS];
#pragma unroll
                for (int r = 0; r < ROWS; ++r) qv[r] = *reinterpret_cast<const int4*>(s_q + (size_t)r * k + (size_t)v * 16);
#pragma unroll
                for (int c = 0; c < MAXC; ++c) {
                    if ((uint32_t)c < cols) {
                        const int4 w = tile[(size_t)c * nvec + v];
#pragma unroll
                        for (int r = 0; r < ROWS; ++r) {
                            int x = acc[c * ROWS + r];
                            x = __dp4a(w.x, qv[r].x, x);
                            x = __dp4a(w.y, qv[r].y, x);
                            x = __dp4a(w.z, qv[r].z, x);
                            x = __dp4a(w.w, qv[r].w, x);
                            acc[c * ROWS + r] = x;
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_empty + 8 * s) : "memory");   // the tile has been consumed
        int* part = s_part + ((i / QS_GROUPS) & 1) * (QS_WARPS * 32) + group * (QS_GROUP_WARPS * 32);
        const int total = qs_reduce<V>(acc, lane);
        if (rlane) part[gwarp * 32 + ridx] = total;
        qs_group_barrier(group);
        if (writer && wc < cols && ok) {
            int sum = 0;
#pragma unroll
            for (int w = 0; w < QS_GROUP_WARPS; ++w) sum += part[w * 32 + gtid];
            if (I4) sum -= 8 * s_sum[wr];
            const uint32_t col = c0 + wc;
            if (zp != 0) atomicOr(status, 16u);   // symmetric form only
            const float sa = s_scale[wr];
            float y = sa == 0.0f ? 0.0f : __fmul_rn(__int2float_rn(sum), __fmul_rn(sa, sc));
            if (residual) y = __fadd_rn(y, res);
            if (act >= 0) y = holo::lut_act_ref(act, y);
            out[(uint64_t)(m0 + wr) * n + col] = y;
        }
    }
}

// ---- the [k, n] weight form with f32 activations ("W8A32", matmul_dequant_float, cpu/float_kernels.rs:596-731) ----
// Two arithmetic definitions, chosen exactly as the CPU backend chooses:
//  * fused (m <= 3, i8, one scale per output column, every zero point 0; cpu/simd.rs:3480-3570): per cell an
//    ascending-k chain acc = fma(a, (f32)q, acc) over the integer levels, then acc * scale[j] once. The last
//    n % 8 columns use multiply-then-add, as the scalar remainder loop does.
//  * dequantize-then-multiply (everything else): w = (f32)(q - zp[ch]) * scale[ch] with ch = (index / inner) %
//    channels (or the per-tensor pair), then the f32 matmul's per-cell chain (fma, multiply-then-add in the
//    n % 8 column tail; cpu/simd.rs:709-802).
// The two factor the scale differently, so their bits differ: the choice must be the reference's. It depends on
// the zero-point values, which live on the device: a one-CTA kernel reduces them to a flag first.
// One thread per four output cells of a row; bit-exact by construction (one chain per cell).
__global__ void zero_points_all_zero_kernel(const int32_t* __restrict__ zps, uint32_t n, uint32_t* flag) {
    holo_pdl_trigger();
    holo_pdl_wait();
    int nonzero = 0;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) nonzero |= zps[i] != 0;
    nonzero = __syncthreads_or(nonzero);
    if (threadIdx.x == 0) *flag = nonzero ? 0u : 1u;
}

__device__ __forceinline__ int read_level(const uint8_t* bq, uint64_t i, int quant_dtype) {
    if (quant_dtype == HOLO_DTYPE_I8) return (int)(int8_t)bq[i];
    if (quant_dtype == HOLO_DTYPE_U8) return (int)bq[i];
    const uint8_t byte = bq[i >> 1];
    const int v = (i & 1) ? (byte >> 4) : (byte & 0x0F);
    return v >= 8 ? v - 16 : v;
}

constexpr int KN_COLS = 4;
__global__ void __launch_bounds__(128)
matmul_dequant_kn_kernel(const float* __restrict__ a, const uint8_t* __restrict__ bq, const float* __restrict__ scales,
                         const int32_t* __restrict__ zps, const float* __restrict__ residual, float* __restrict__ out, uint32_t m, uint32_t k,
                         uint32_t n, uint32_t channels, uint32_t inner, int quant_dtype, float scale, int32_t zp, int act, int fused_eligible,
                         const uint32_t* __restrict__ zero_flag) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint32_t j0 = (blockIdx.x * blockDim.x + threadIdx.x) * KN_COLS, i = blockIdx.y;
    if (j0 >= n || i >= m) return;
    const bool per_ch = scales != nullptr;
    const bool fused = fused_eligible && *zero_flag != 0;
    const uint32_t tail_begin = n - (n % 8);
    float acc[KN_COLS];
#pragma unroll
    for (int c = 0; c < KN_COLS; ++c) acc[c] = 0.0f;
    const float* arow = a + (uint64_t)i * k;
    for (uint32_t kk = 0; kk < k; ++kk) {
        const float av = arow[kk];
#pragma unroll
        for (int c = 0; c < KN_COLS; ++c) {
            const uint32_t j = j0 + c;
            if (j >= n) break;
            const uint64_t idx = (uint64_t)kk * n + j;
            const int q = read_level(bq, idx, quant_dtype);
            float w;
            if (fused) {
                w = (float)q;
            } else if (per_ch) {
                const uint32_t ch = (uint32_t)((idx / inner) % channels);
                w = __fmul_rn((float)(q - zps[ch]), scales[ch]);
            } else {
                w = __fmul_rn((float)(q - zp), scale);
            }
            acc[c] = j < tail_begin ? __fmaf_rn(av, w, acc[c]) : __fadd_rn(acc[c], __fmul_rn(av, w));
        }
    }
#pragma unroll
    for (int c = 0; c < KN_COLS; ++c) {
        const uint32_t j = j0 + c;
        if (j >= n) break;
        float y = fused ? __fmul_rn(acc[c], scales[j]) : acc[c];
        const uint64_t o = (uint64_t)i * n + j;
        if (residual) y = __fadd_rn(y, residual[o]);
        if (act >= 0) y = holo::lut_act_ref(act, y);
        out[o] = y;
    }
}

template <int ROWS, bool I4>
cudaError_t launch_stream(holo_b200_ctx* ctx, uint32_t grid, size_t smem, const float* a, const int8_t* bq, const float* scales,
                          const int32_t* zero_points, const float* residual, float* out, uint32_t m0, uint32_t rows, uint32_t k,
                          uint32_t n, uint32_t cols_per_tile, uint32_t stages, int act) {
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        cudaError_t e = cudaFuncSetAttribute(matmul_w8a8_stream_kernel<ROWS, I4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)QS_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        configured_device = ctx->device;
    }
    return holo_launch_kernel(ctx, matmul_w8a8_stream_kernel<ROWS, I4>, dim3(grid), dim3((QS_WARPS + 1) * 32), smem, 1, a, bq, scales, zero_points,
                              residual, out, m0, rows, k, n, cols_per_tile, stages, act, ctx->dev_status);
}

}  // namespace

int32_t holo_launch_matmul_e8cb_omajor(holo_b200_ctx* ctx, const float* a, const uint8_t* bq, const int8_t* codebook, const float* scales,
                                       const int32_t* zero_points, const float* residual, float* out, uint32_t m, uint32_t k, uint32_t n, int act) {
    if (m == 0 || k == 0 || n == 0) return HOLO_OK;
    const uint32_t kpad = (k + 15u) & ~15u;
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        HOLO_CUDA(cudaFuncSetAttribute(matmul_e8cb_omajor_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
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
        HOLO_CUDA(holo_launch_kernel(ctx, matmul_e8cb_omajor_kernel, dim3(grid), dim3(QG_WARPS * 32), (size_t)take * kpad, 1, a, bq, codebook, scales,
                                     zero_points, residual, out, m0, take, k, n, act, ctx->dev_status));
        ctx->launches++;
    }
    return HOLO_OK;
}

int32_t holo_launch_matmul_w8a8_omajor(holo_b200_ctx* ctx, const float* a, const int8_t* bq, const float* scales, const int32_t* zero_points,
                                       const float* residual, float* out, uint32_t m, uint32_t k, uint32_t n, int act, bool i4) {
    if (m == 0 || k == 0 || n == 0) return HOLO_OK;
    const uint32_t kw = i4 ? k >> 1 : k;   // bytes of one weight column
    const bool streamable = (kw & 15u) == 0 && kw <= QS_STAGE_BYTES && ((uintptr_t)bq & 15u) == 0;
    if (i4 && (!streamable || (size_t)k > 64 * 1024))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: the packed-i4 form is served for k a multiple of 32 up to 32768 and a 16-byte aligned weight");
    if (streamable && (i4 || !getenv("HOLO_W8A8_NO_STREAM"))) {
        uint32_t per = QG_MAX_ROWS;   // rows per launch: what fits beside the ring in shared memory
        while (per > 1 && qs_smem_bytes(per, k, QS_MIN_STAGES) > QS_SMEM_LIMIT) per >>= 1;
        for (uint32_t m0 = 0; m0 < m; m0 += per) {
            const uint32_t take = m - m0 < per ? m - m0 : per;
            const uint32_t rt = take > 4 ? 8 : take > 2 ? 4 : take;
            uint32_t cols_per_tile = QS_STAGE_BYTES / kw;
            if (cols_per_tile > (uint32_t)qs_max_cols((int)rt, i4)) cols_per_tile = (uint32_t)qs_max_cols((int)rt, i4);
            const uint32_t ntiles = (n + cols_per_tile - 1) / cols_per_tile;
            const uint32_t grid = ntiles < (uint32_t)ctx->sm_count ? ntiles : (uint32_t)ctx->sm_count;
            uint32_t stages = QS_MAX_STAGES;
            while (stages > QS_MIN_STAGES && qs_smem_bytes(rt, k, stages) > QS_SMEM_LIMIT) --stages;
            const size_t smem = qs_smem_bytes(rt, k, stages);
#define QS_LAUNCH(R, Q) launch_stream<R, Q>(ctx, grid, smem, a, bq, scales, zero_points, residual, out, m0, take, k, n, cols_per_tile, stages, act)
            cudaError_t e = i4 ? (rt == 8 ? QS_LAUNCH(8, true) : rt == 4 ? QS_LAUNCH(4, true) : rt == 2 ? QS_LAUNCH(2, true) : QS_LAUNCH(1, true))
                               : (rt == 8 ? QS_LAUNCH(8, false) : rt == 4 ? QS_LAUNCH(4, false) : rt == 2 ? QS_LAUNCH(2, false) : QS_LAUNCH(1, false));
#undef QS_LAUNCH
            HOLO_CUDA(e);
            ctx->launches++;
        }
        return HOLO_OK;
    }
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


// MatMulDequant over a [k, n] weight with f32 activations (see matmul_dequant_kn_kernel). `scales` / `zero_points`
// null = per-tensor (scale, zero_point).
int32_t holo_launch_matmul_dequant_kn(holo_b200_ctx* ctx, const float* a, const uint8_t* bq, const float* scales, const int32_t* zero_points,
                                      const float* residual, float* out, uint32_t m, uint32_t k, uint32_t n, uint32_t channels, uint32_t inner,
                                      uint8_t quant_dtype, float scale, int32_t zero_point, int act) {
    if (m == 0 || k == 0 || n == 0) return HOLO_OK;
    if (m > 65535) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: m %u on the [k,n] path", m);
    const bool per_ch = scales != nullptr;
    if (inner == 0) inner = 1;
    // FUSED_W8A32_MAX_M = 3 (kernel_call.rs decode_gate)
    const int fused_eligible = per_ch && quant_dtype == HOLO_DTYPE_I8 && m <= 3 && channels == n && inner == 1;
    uint32_t* flag = ctx->dev_status + 16;   // a spare word of the status block
    if (fused_eligible) {
        HOLO_CUDA(holo_launch_kernel(ctx, zero_points_all_zero_kernel, dim3(1), dim3(256), 0, 1, zero_points, n, flag));
        ctx->launches++;
    }
    const uint32_t per_cta = 128 * KN_COLS;
    HOLO_CUDA(holo_launch_kernel(ctx, matmul_dequant_kn_kernel, dim3((n + per_cta - 1) / per_cta, m), dim3(128), 0, 1, a, bq, scales, zero_points, residual,
                                 out, m, k, n, channels, inner, (int)quant_dtype, scale, zero_point, act, fused_eligible, (const uint32_t*)flag));
    ctx->launches++;
    return HOLO_OK;
}
