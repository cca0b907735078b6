// Single-token decode attention over an int8 KV cache (and the general-shape form).
//
// Replaces decode_attention_valid_float (crates/hologram-compute/src/cpu/float_kernels.rs:4192-4307,
// row kernel :3834-3883) for the quantized-cache composition
//   Cast(q) -> Dequantize(K, V per cache row) -> DecodeAttentionValid(f32) -> Cast(out).
//
// The tiled kernel is HBM-bound: every K/V code byte is read once per GQA group. Design:
//   * persistent grid (2 CTAs per SM): the (plane, 128-key tile) pairs, plane = (batch, kv head),
//     form one list in plane-major order and every CTA walks an equal contiguous share of it
//     (flash-decoding split-KV with no idle tail and a ring that never drains); a plane held by one
//     CTA is finished by it, a plane shared by several goes through partial (max, sum, context)
//     triples in a scratch buffer that the last sharer to count in merges (nobody waits).
//   * a producer warp feeds a 3-stage ring with TMA (cp.async.bulk.tensor, 128B swizzle):
//     K codes, V codes, K scales, V scales per stage; mbarrier full/empty pairs, bounded waits.
//   * dequantisation is never materialised. q is split into three signed base-256 digits per
//     head (rows of one m16 tile), so q.k is an exact integer dot on the int8 tensor-core path
//     (mma.sync m16n8k32 s8) fed straight from the swizzled tile by ldmatrix; the per-row K
//     scale multiplies the score. Softmax weights times the per-row V scale are likewise cut
//     into three unsigned digits and multiplied with the raw V codes (u8 x s8 MMA), the V tile
//     being transposed on the fly by ldmatrix.trans + byte permutes. Integer accumulators are
//     folded into f32 only when the running maximum (or the digit scale) has to change.
#include <cuda.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "attention_generic.cuh"
#include "common.h"
#include "numerics.cuh"

namespace {

constexpr int TK = 128;           // keys per tile
constexpr int HD = 128;           // head_dim served by the tiled kernel
#ifndef HOLO_ATTN_STAGES
#define HOLO_ATTN_STAGES 3
#endif
#ifndef HOLO_ATTN_MINB
#define HOLO_ATTN_MINB 2
#endif
constexpr int STAGES = HOLO_ATTN_STAGES;
constexpr int CONSUMER_WARPS = 4;
constexpr int FA_THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int MAXG = 4;           // query heads per kv head served by the tiled kernel
constexpr uint32_t STAGE_K = 0, STAGE_V = TK * HD, STAGE_SK = 2 * TK * HD, STAGE_SV = 2 * TK * HD + TK * 4;
constexpr uint32_t STAGE_BYTES = 2 * TK * HD + 2 * TK * 4;  // 33792
constexpr uint32_t SMEM_Q = STAGES * STAGE_BYTES;            // 16 x 128 B digit tile
constexpr uint32_t SMEM_MISC = SMEM_Q + 16 * HD;             // cq[4], bad[4], abort, barriers
constexpr uint32_t SMEM_MERGE = SMEM_MISC + 256;             // 4 warps x 4 heads x (128 + 2) f32
constexpr uint32_t SMEM_TOTAL = SMEM_MERGE + CONSUMER_WARPS * MAXG * (HD + 2) * 4 + 1024;  // + alignment slack
constexpr uint32_t WAIT_LIMIT = 1u << 20;
constexpr float LOG2E = 1.4426950408889634f;

struct FaParams {
    const void* q;
    const int8_t *k_new, *v_new;
    const float *k_new_s, *v_new_s;
    const uint32_t* valid_len;
    void* out;
    float* part_o;   // [plane][slot][MAXG][HD]
    float* part_ml;  // [plane][slot][MAXG][2]
    uint32_t* status;
    uint32_t* arrivals;  // [planes] zero between launches: CTAs that have stored their partial of a shared plane
    uint32_t past, G, planes, max_slots, box_rows;
    float scale_div;
    int dtype;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait: gives up after WAIT_LIMIT polls, raises the abort flag and a status bit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (it > 64) __nanosleep(64);
    }
    *abort_flag = 1;
    atomicOr(status, 2u);
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_s8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Byte address of (row, 16-byte chunk) inside a [rows][128 B] tile written by TMA with the
// 128-byte swizzle (chunk index XOR row mod 8); the tile base is 1024-byte aligned.
__device__ __forceinline__ uint32_t swz(uint32_t base, uint32_t row, uint32_t chunk) {
    return base + row * 128u + ((chunk ^ (row & 7u)) << 4);
}
__device__ __forceinline__ float exp2_guard(float s, float m) {
    // exp(s - m) for a finite or -inf score s against reference m (m may be -inf before the
    // first fold, which must yield +inf so that the fold triggers).
    if (s == -INFINITY) return 0.0f;
    return exp2f((s - m) * LOG2E);
}

// Ownership of the global tile list: CTA c of n takes tiles [total*c/n, total*(c+1)/n).
__device__ __forceinline__ uint32_t fa_start(uint32_t c, uint32_t total, uint32_t nctas) {
    return (uint32_t)(((uint64_t)total * c) / nctas);
}
// The CTA whose share holds tile g: the largest c with fa_start(c) <= g, i.e. c < (g + 1) n / total.
__device__ __forceinline__ uint32_t fa_owner(uint32_t g, uint32_t total, uint32_t nctas) {
    return (uint32_t)((((uint64_t)g + 1) * nctas - 1) / total);
}

// Fold the stored partials of slots [from, nsl) of one plane onto the running (max, sum, context)
// triples of element c of each head, in slot order, and write the plane's result. Four slots per
// round, with all of a round's loads issued before the first use (each is an L2 round trip).
__device__ __forceinline__ void merge_slots(const FaParams& p, uint32_t plane, uint32_t first, uint32_t from, uint32_t nsl,
                                            uint32_t total, uint32_t nctas, uint32_t G, uint32_t c, float (&M)[MAXG],
                                            float (&L)[MAXG], float (&O)[MAXG]) {
    for (uint32_t s0 = from; s0 < nsl; s0 += 4) {
        float2 ml[4][MAXG];
        float ov[4][MAXG];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t sl = s0 + j;
            // a CTA whose share of the list is empty (more CTAs than tiles) stored nothing
            const bool live = sl < nsl && !(nctas > total && fa_start(first + sl, total, nctas) == fa_start(first + sl + 1, total, nctas));
#pragma unroll
            for (int gg = 0; gg < MAXG; ++gg) {
                ml[j][gg] = make_float2(-INFINITY, 0.0f);
                ov[j][gg] = 0.0f;
                if (live && (uint32_t)gg < G) {
                    const uint64_t pidx = ((uint64_t)plane * p.max_slots + sl) * MAXG + gg;
                    ml[j][gg] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + pidx * 2));
                    ov[j][gg] = __ldcg(p.part_o + pidx * HD + c);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int gg = 0; gg < MAXG; ++gg) {
                const float wm = ml[j][gg].x;
                if (wm != -INFINITY) {
                    const float nm = fmaxf(M[gg], wm);
                    const float fo = exp2_guard(M[gg], nm), fn = exp2f((wm - nm) * LOG2E);
                    L[gg] = fmaf(ml[j][gg].y, fn, L[gg] * fo);
                    O[gg] = fmaf(ov[j][gg], fn, O[gg] * fo);
                    M[gg] = nm;
                }
            }
    }
#pragma unroll
    for (int gg = 0; gg < MAXG; ++gg)
        if ((uint32_t)gg < G) holo::store_float(p.out, ((uint64_t)plane * G + gg) * HD + c, O[gg] / fmaxf(L[gg], 1e-30f), p.dtype);
}

// Persistent kernel. The work is the list of (plane, tile) pairs in plane-major order, every
// plane contributing ceil(visible/128) cache tiles plus one tile for this step's new row. Each
// CTA owns an equal contiguous share of that list, so its TMA ring never drains between planes
// and no wave of CTAs ends with idle SMs. A share covers parts of a few planes ("segments"); for
// each segment the consumers rebuild the query digits, run the tiles, merge their four running
// (max, sum, context) triples, and either write the plane's result (the CTA had the whole plane)
// or store a partial and count in on the plane's arrival counter; the CTA that counts in last
// merges the plane's partials. Nobody waits for anybody: a CTA that is not last simply goes on.
__global__ void __launch_bounds__(FA_THREADS, HOLO_ATTN_MINB)
decode_attention_q8_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                           const __grid_constant__ CUtensorMap map_ks, const __grid_constant__ CUtensorMap map_vs,
                           const FaParams p) {
    holo_pdl_trigger();
    holo_pdl_wait();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    float* s_cq = reinterpret_cast<float*>(sm + SMEM_MISC);            // [4]
    uint32_t* s_bad = reinterpret_cast<uint32_t*>(sm + SMEM_MISC + 16);  // [4]
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(sm + SMEM_MISC + 32);
    uint32_t* s_fast = reinterpret_cast<uint32_t*>(sm + SMEM_MISC + 36);
    uint32_t* s_last = reinterpret_cast<uint32_t*>(sm + SMEM_MISC + 192);  // [9]
    float* s_red = reinterpret_cast<float*>(sm + SMEM_MISC + 64);       // [4 warps][4 heads]
    const uint32_t bar_full = base + SMEM_MISC + 128, bar_empty = bar_full + 8 * STAGES;
    float* mo = reinterpret_cast<float*>(sm + SMEM_MERGE);  // [warp][head][HD]
    float* mml = mo + CONSUMER_WARPS * MAXG * HD;            // [warp][head][2]

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t G = p.G, nctas = gridDim.x, cta = blockIdx.x;
    const uint32_t vis_past = min(*p.valid_len, p.past);
    const uint32_t tiles_past = (vis_past + TK - 1) / TK;
    const uint32_t T = tiles_past + 1;  // + the tile holding this step's new row
    const uint32_t total = p.planes * T;
    const uint32_t g0 = fa_start(cta, total, nctas), g1 = fa_start(cta + 1, total, nctas);

    // an earlier launch gave up on a wait: do not start
    if (*reinterpret_cast<volatile uint32_t*>(p.status) & 2u) return;
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, CONSUMER_WARPS);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer warp ----------------
        const uint32_t tx_bytes = p.box_rows * HD * 2 + p.box_rows * 4 * 2;
        uint32_t it = 0;
        for (uint32_t g = g0; g < g1; ++g, ++it) {
            const uint32_t s = it % STAGES, use = it / STAGES;
            const uint32_t plane = g / T, t = g % T;
            if (use > 0) {
                bool ok = true;
                if (lane == 0) ok = mbar_wait(bar_empty + 8 * s, (use - 1) & 1, s_abort, p.status);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            const uint32_t st = base + s * STAGE_BYTES;
            if (t < tiles_past) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(bar_full + 8 * s, tx_bytes);
                    tma_load_3d(st + STAGE_K, &map_k, 0, (int)(t * TK), (int)plane, bar_full + 8 * s);
                    tma_load_3d(st + STAGE_V, &map_v, 0, (int)(t * TK), (int)plane, bar_full + 8 * s);
                    tma_load_2d(st + STAGE_SK, &map_ks, (int)(t * TK), (int)plane, bar_full + 8 * s);
                    tma_load_2d(st + STAGE_SV, &map_vs, (int)(t * TK), (int)plane, bar_full + 8 * s);
                }
            } else {
                // the new row of this step: row 0 of the tile (row 0 is unaffected by the swizzle)
                uint8_t* sp = sm + s * STAGE_BYTES;
                if (lane < 8) reinterpret_cast<uint4*>(sp + STAGE_K)[lane] = reinterpret_cast<const uint4*>(p.k_new + (uint64_t)plane * HD)[lane];
                else if (lane < 16) reinterpret_cast<uint4*>(sp + STAGE_V)[lane - 8] = reinterpret_cast<const uint4*>(p.v_new + (uint64_t)plane * HD)[lane - 8];
                else if (lane == 16) reinterpret_cast<float*>(sp + STAGE_SK)[0] = p.k_new_s[plane];
                else if (lane == 17) reinterpret_cast<float*>(sp + STAGE_SV)[0] = p.v_new_s[plane];
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * s);
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    const uint32_t r = lane >> 2, i = lane & 3;
    const bool hi_group = r >= 4;       // lanes holding digit L1 (and the zero row)
    const uint32_t g = r & 3;           // head served by this lane
    const uint32_t selA = hi_group ? 0x0051u : 0x0062u;  // digit byte of (x, y): L1 = byte 1, L0 = byte 2
    const uint32_t selB = hi_group ? 0x0073u : 0x0040u;  // zero byte 3, or L2 = byte 0
    int acc[8][2][4];
    float of[32];
    float m_ref, l_sum, sref, inv_sref;
    uint32_t since_fold;
    uint32_t qa[4][4];
    float cq;

    auto fold = [&]() {
        if (sref != 0.0f) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int eo = e & 1, nn = e >> 1;
                    float v = hi_group ? __int2float_rn(acc[c][eo][nn]) * 256.0f
                                       : fmaf(__int2float_rn(acc[c][eo][nn]), 65536.0f, __int2float_rn(acc[c][eo][2 + nn]));
                    of[c * 4 + e] = fmaf(v, inv_sref, of[c * 4 + e]);
                }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
#pragma unroll
            for (int e = 0; e < 2; ++e)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[c][e][x] = 0;
        since_fold = 0;
    };


    uint32_t it = 0;
    bool aborted = false;
    uint32_t gt = g0;
    uint32_t npend = 0, pend_plane[2], pend_first[2], pend_last[2], pend_sharers[2], pend_before[2];  // thread 0 only
    while (gt < g1) {
        const uint32_t plane = gt / T;
        const uint32_t seg_end = min(g1, (plane + 1) * T);
        // the plane's first sharer looks at the arrival counter now and uses the value when the
        // segment ends, so the round trip is hidden behind the segment's tiles
        uint32_t probe = 0;
        if (tid == 0 && fa_owner(plane * T, total, nctas) == cta && fa_owner(plane * T + T - 1, total, nctas) != cta)
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(probe) : "l"(p.arrivals + plane) : "memory");
        // ---- query digits of this plane: q = (L0*65536 + L1*256 + L2) * 2^(ex-21), one row of
        // the m16 tile per (head, digit): rows g, 4+g, 8+g hold L0, L1, L2 of head g; rows 12.. zero.
        {
            int8_t* sq = reinterpret_cast<int8_t*>(sm + SMEM_Q);
            float qv[MAXG];
#pragma unroll
            for (int gg = 0; gg < MAXG; ++gg) {
                qv[gg] = (uint32_t)gg < G ? holo::load_float(p.q, ((uint64_t)plane * G + gg) * HD + tid, p.dtype) : 0.0f;
                float a = fabsf(qv[gg]);
                for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
                // NaN elements are dropped by fmaxf; detect them separately
                uint32_t nanbit = __any_sync(0xffffffffu, qv[gg] != qv[gg]);
                if (lane == 0) s_red[warp * 4 + gg] = nanbit ? INFINITY : a;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
            for (int gg = 0; gg < MAXG; ++gg) {
                float amax = fmaxf(fmaxf(s_red[gg], s_red[4 + gg]), fmaxf(s_red[8 + gg], s_red[12 + gg]));
                uint32_t be = (__float_as_uint(amax) >> 23) & 0xffu;
                int L0 = 0, L1 = 0, L2 = 0;
                float cqv = 0.0f;
                uint32_t bad = 0;
                if (be == 255u) {
                    bad = 1;  // inf / NaN in q: the reference yields NaN for the whole head
                } else if (be != 0u) {
                    int ex = (int)be - 127;  // amax < 2^(ex+1)
                    int qi = __float2int_rn(scalbnf(qv[gg], 21 - ex));  // |qi| < 2^22 keeps L0 within int8
                    L2 = ((qi + 128) & 255) - 128;
                    int q1 = (qi - L2) >> 8;
                    L1 = ((q1 + 128) & 255) - 128;
                    L0 = (q1 - L1) >> 8;
                    cqv = scalbnf(1.0f, ex - 21) / p.scale_div;
                }
                sq[(gg)*HD + tid] = (int8_t)L0;
                sq[(4 + gg) * HD + tid] = (int8_t)L1;
                sq[(8 + gg) * HD + tid] = (int8_t)L2;
                sq[(12 + gg) * HD + tid] = 0;
                if (tid == 0) {
                    s_cq[gg] = cqv;
                    s_bad[gg] = bad;
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            cq = s_cq[g];
            const uint32_t* sq32 = reinterpret_cast<const uint32_t*>(sm + SMEM_Q);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                qa[ks][0] = sq32[(r * HD + 32 * ks + 4 * i) >> 2];
                qa[ks][1] = sq32[((r + 8) * HD + 32 * ks + 4 * i) >> 2];
                qa[ks][2] = sq32[(r * HD + 32 * ks + 16 + 4 * i) >> 2];
                qa[ks][3] = sq32[((r + 8) * HD + 32 * ks + 16 + 4 * i) >> 2];
            }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
#pragma unroll
            for (int e = 0; e < 2; ++e)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[c][e][x] = 0;
#pragma unroll
        for (int x = 0; x < 32; ++x) of[x] = 0.0f;
        m_ref = -INFINITY;
        l_sum = 0.0f;
        sref = 0.0f;
        inv_sref = 0.0f;
        since_fold = 0;

        for (; gt < seg_end; ++gt, ++it) {
            const uint32_t s = it % STAGES, use = it / STAGES;
            const uint32_t t = gt % T;
            // after a failed wait the warp keeps walking (so that every barrier below is still
            // reached by all four warps) but touches no tile
            if (!aborted && !mbar_wait(bar_full + 8 * s, use & 1, s_abort, p.status)) aborted = true;
            const uint32_t st = base + s * STAGE_BYTES;
            const uint8_t* sp = sm + s * STAGE_BYTES;
            // keys of this warp: tile rows 32*warp .. +31; number of visible rows in the tile
            const uint32_t limit = t < tiles_past ? min((uint32_t)TK, vis_past - t * TK) : 1u;
            const uint32_t row0 = warp * 32;
            if (!aborted && row0 < limit) {
                // ---- scores: S[(head,digit)][key] = sum_c Qdigit * Kcode (exact i32) ----
                int sacc[4][4];
    #pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
    #pragma unroll
                    for (int x = 0; x < 4; ++x) sacc[nt][x] = 0;
    #pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t kb[4];
                        ldsm_x4(kb, swz(st + STAGE_K, row0 + 8 * nt + (lane & 7), 4 * half + (lane >> 3)));
                        mma_s8s8(sacc[nt], qa[2 * half], kb[0], kb[1]);
                        mma_s8s8(sacc[nt], qa[2 * half + 1], kb[2], kb[3]);
                    }
                }
                const float* sk = reinterpret_cast<const float*>(sp + STAGE_SK);
                const float* sv = reinterpret_cast<const float*>(sp + STAGE_SV);
                float sc[8], svv[8];
                float mt = -INFINITY;
    #pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const uint32_t key = row0 + 8 * nt + 2 * i;
                    const float2 k2 = *reinterpret_cast<const float2*>(sk + key);
                    const float2 v2 = *reinterpret_cast<const float2*>(sv + key);
    #pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        float part = hi_group ? __int2float_rn(sacc[nt][e]) * 256.0f
                                              : fmaf(__int2float_rn(sacc[nt][e]), 65536.0f, __int2float_rn(sacc[nt][2 + e]));
                        float full = part + __shfl_xor_sync(0xffffffffu, part, 16);
                        float kscale = e ? k2.y : k2.x;
                        float sval = full * (kscale * cq);
                        float vscale = e ? v2.y : v2.x;
                        if (key + e >= limit) {  // unrealized row: whatever bytes it holds never count
                            sval = -INFINITY;
                            vscale = 0.0f;
                        }
                        sc[nt * 2 + e] = sval;
                        svv[nt * 2 + e] = vscale;
                        mt = fmaxf(mt, sval);
                    }
                }
                mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
                mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
                // ---- weights relative to the running reference, scaled for digit extraction ----
                float pe[8], ps[8];
                float pmax = 0.0f;
    #pragma unroll
                for (int x = 0; x < 8; ++x) {
                    pe[x] = exp2_guard(sc[x], m_ref);
                    ps[x] = pe[x] * svv[x] * sref;
                    pmax = fmaxf(pmax, ps[x] != ps[x] ? INFINITY : ps[x]);
                }
                pmax = fmaxf(pmax, __shfl_xor_sync(0xffffffffu, pmax, 1));
                pmax = fmaxf(pmax, __shfl_xor_sync(0xffffffffu, pmax, 2));
                const bool need = !(pmax < 16777215.0f) || mt > m_ref + 60.0f || sref == 0.0f || since_fold >= 1024;
                if (__any_sync(0xffffffffu, need)) {
                    fold();
                    const float m_new = fmaxf(m_ref, mt);
                    const float alpha = m_ref == -INFINITY ? 0.0f : exp2f((m_ref - m_new) * LOG2E);
    #pragma unroll
                    for (int x = 0; x < 32; ++x) of[x] *= alpha;
                    l_sum *= alpha;
                    m_ref = m_new;
                    float pm = 0.0f;
    #pragma unroll
                    for (int x = 0; x < 8; ++x) {
                        pe[x] = exp2_guard(sc[x], m_ref);
                        float w = pe[x] * svv[x];
                        pm = fmaxf(pm, w);
                    }
                    pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 1));
                    pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 2));
                    int sexp = 0;
                    const uint32_t pbe = (__float_as_uint(pm) >> 23) & 0xffu;
                    if (pbe != 0u && pbe != 255u) sexp = 15 - ((int)pbe - 127);
                    sexp = max(-100, min(100, sexp));
                    sref = __uint_as_float((uint32_t)(127 + sexp) << 23);
                    inv_sref = __uint_as_float((uint32_t)(127 - sexp) << 23);
    #pragma unroll
                    for (int x = 0; x < 8; ++x) ps[x] = fminf(pe[x] * svv[x] * sref, 16777215.0f);
                }
                uint32_t pi[8];
    #pragma unroll
                for (int x = 0; x < 8; ++x) {
                    l_sum += pe[x];
                    pi[x] = __float2uint_rn(fmaxf(ps[x], 0.0f));
                }
                uint32_t pa[4];
                pa[0] = __byte_perm(__byte_perm(pi[0], pi[1], selA), __byte_perm(pi[2], pi[3], selA), 0x5410);
                pa[1] = __byte_perm(__byte_perm(pi[0], pi[1], selB), __byte_perm(pi[2], pi[3], selB), 0x5410);
                pa[2] = __byte_perm(__byte_perm(pi[4], pi[5], selA), __byte_perm(pi[6], pi[7], selA), 0x5410);
                pa[3] = __byte_perm(__byte_perm(pi[4], pi[5], selB), __byte_perm(pi[6], pi[7], selB), 0x5410);
                // ---- context: O[(head,digit)][c] += sum_key Pdigit * Vcode ----
    #pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    uint32_t vr[4];
                    ldsm_x4_trans(vr, swz(st + STAGE_V, row0 + 8 * (lane >> 3) + (lane & 7), ch));
                    mma_u8s8(acc[ch][0], pa, __byte_perm(vr[0], vr[1], 0x6420), __byte_perm(vr[2], vr[3], 0x6420));
                    mma_u8s8(acc[ch][1], pa, __byte_perm(vr[0], vr[1], 0x7531), __byte_perm(vr[2], vr[3], 0x7531));
                }
                ++since_fold;
            }
            __syncwarp();
            if (lane == 0 && !aborted) mbar_arrive(bar_empty + 8 * s);
        }
        fold();
        // ---- merge the four warps' triples; finish the plane or publish this segment's partial ----
        l_sum += __shfl_xor_sync(0xffffffffu, l_sum, 1);
        l_sum += __shfl_xor_sync(0xffffffffu, l_sum, 2);
#pragma unroll
        for (int x = 0; x < 32; ++x) of[x] += __shfl_xor_sync(0xffffffffu, of[x], 16);
        if (!hi_group) {
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<float4*>(mo + ((warp * MAXG + g) * HD + 16 * c + 4 * i)) =
                    make_float4(of[c * 4 + 0], of[c * 4 + 1], of[c * 4 + 2], of[c * 4 + 3]);
            if (i == 0) {
                mml[(warp * MAXG + g) * 2 + 0] = m_ref;
                mml[(warp * MAXG + g) * 2 + 1] = l_sum;
            }
        }
        // CTAs first..last hold parts of this plane; those with a non-empty share are its sharers
        const uint32_t first = fa_owner(plane * T, total, nctas), last = fa_owner(plane * T + T - 1, total, nctas);
        uint32_t sharers = last - first + 1;
        if (nctas > total) {
            sharers = 0;
            for (uint32_t cc = first; cc <= last; ++cc) sharers += fa_start(cc, total, nctas) != fa_start(cc + 1, total, nctas);
        }
        if (tid == 0) *s_fast = sharers > 1 && cta == first && probe + 1 == sharers;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!aborted && !*s_abort) {
            // CTAs first..last share this plane; each but one stores a partial and counts in on the
            // plane's arrival counter, and one CTA merges. The first sharer reaches its part last
            // (it is the tail of its share), so it normally finds everybody else counted in (the
            // probe taken when the segment began) and merges their partials on top of its own
            // triple without a round trip of its own. Otherwise it publishes like the others, and
            // whoever counts in last merges. Either way the merge runs over the slots in order on
            // the same f32 values, so the result does not depend on who merged.
            const uint32_t c = tid;  // 0..127
            float M[MAXG], L[MAXG], O[MAXG];
#pragma unroll
            for (int gg = 0; gg < MAXG; ++gg) {
                M[gg] = -INFINITY;
                L[gg] = 0.0f;
                O[gg] = 0.0f;
                if ((uint32_t)gg < G) {
#pragma unroll
                    for (int w = 0; w < CONSUMER_WARPS; ++w) M[gg] = fmaxf(M[gg], mml[(w * MAXG + gg) * 2]);
#pragma unroll
                    for (int w = 0; w < CONSUMER_WARPS; ++w) {
                        float wm = mml[(w * MAXG + gg) * 2];
                        if (wm != -INFINITY) {
                            float f = exp2f((wm - M[gg]) * LOG2E);
                            L[gg] = fmaf(mml[(w * MAXG + gg) * 2 + 1], f, L[gg]);
                            O[gg] = fmaf(mo[(w * MAXG + gg) * HD + c], f, O[gg]);
                        }
                    }
                    if (s_bad[gg]) { O[gg] = NAN; L[gg] = 1.0f; M[gg] = 0.0f; }
                }
            }
            if (sharers == 1) {
#pragma unroll
                for (int gg = 0; gg < MAXG; ++gg)
                    if ((uint32_t)gg < G)
                        holo::store_float(p.out, ((uint64_t)plane * G + gg) * HD + c, O[gg] / fmaxf(L[gg], 1e-30f), p.dtype);
            } else if (*s_fast) {
                // the probe was an acquire load by thread 0 and a barrier lies between it and here,
                // so the others' partials are visible to every thread of the CTA (read from L2)
                merge_slots(p, plane, first, 1, last - first + 1, total, nctas, G, c, M, L, O);
                if (tid == 0) p.arrivals[plane] = 0;  // everybody else has counted in: ready for the next launch
            } else {
                const uint32_t slot = cta - first;
#pragma unroll
                for (int gg = 0; gg < MAXG; ++gg)
                    if ((uint32_t)gg < G) {
                        const uint64_t pidx = ((uint64_t)plane * p.max_slots + slot) * MAXG + gg;
                        p.part_o[pidx * HD + c] = O[gg];
                        if (c == 0) *reinterpret_cast<float2*>(p.part_ml + pidx * 2) = make_float2(M[gg], L[gg]);
                    }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (tid == 0 && npend < 2) {
                    // the count comes back while the next segment streams; it is read at the end
                    pend_before[npend] = atomicAdd(p.arrivals + plane, 1u);
                    pend_plane[npend] = plane;
                    pend_first[npend] = first;
                    pend_last[npend] = last;
                    pend_sharers[npend] = sharers;
                    ++npend;
                }
            }
        }
        // the merge area, the digit tile and s_red are rewritten by the next segment
        asm volatile("bar.sync 1, 128;" ::: "memory");
    }

    // ---- a CTA that counted in last on a plane merges that plane's partials ----
    if (tid == 0) {
        s_last[0] = s_last[1] = 0;
        s_last[2] = npend;
        for (uint32_t k = 0; k < npend; ++k) {
            const uint32_t is_last = pend_before[k] + 1 == pend_sharers[k];
            if (is_last) p.arrivals[pend_plane[k]] = 0;
            s_last[k] = is_last;
            s_last[3 + 3 * k] = pend_plane[k];
            s_last[4 + 3 * k] = pend_first[k];
            s_last[5 + 3 * k] = pend_last[k];
        }
        __threadfence();  // acquire side of the counts read above, for the whole CTA through the barrier
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (aborted || *s_abort) return;
    const uint32_t n_published = s_last[2];
    for (uint32_t k = 0; k < n_published; ++k) {
        if (!s_last[k]) continue;
        const uint32_t plane = s_last[3 + 3 * k], first = s_last[4 + 3 * k], last = s_last[5 + 3 * k];
        float M[MAXG], L[MAXG], O[MAXG];
#pragma unroll
        for (int gg = 0; gg < MAXG; ++gg) { M[gg] = -INFINITY; L[gg] = 0.0f; O[gg] = 0.0f; }
        merge_slots(p, plane, first, 0, last - first + 1, total, nctas, G, tid, M, L, O);
    }
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    return fn;
}

int32_t make_codes_map(CUtensorMap* map, const void* ptr, uint32_t past, uint32_t planes, uint32_t box_rows) {
    cuuint64_t dims[3] = {HD, past, planes};
    cuuint64_t strides[2] = {HD, (cuuint64_t)HD * past};
    cuuint32_t box[3] = {HD, box_rows, 1};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, es,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: cuTensorMapEncodeTiled (codes) returned %d", (int)r);
    return HOLO_OK;
}
int32_t make_scales_map(CUtensorMap* map, const void* ptr, uint32_t past, uint32_t planes, uint32_t box_rows) {
    cuuint64_t dims[2] = {past, planes};
    cuuint64_t strides[1] = {(cuuint64_t)past * 4};
    cuuint32_t box[2] = {box_rows, 1};
    cuuint32_t es[2] = {1, 1};
    CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, es,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: cuTensorMapEncodeTiled (scales) returned %d", (int)r);
    return HOLO_OK;
}

// Grid of the persistent kernel: HOLO_ATTN_MINB CTAs per SM (all co-resident), never more than
// there are tiles. A plane is then shared by at most nctas / planes + 2 CTAs.
uint32_t persistent_ctas(uint32_t tiles_per_plane, uint32_t planes, int sm_count) {
    uint64_t want = (uint64_t)HOLO_ATTN_MINB * (uint32_t)sm_count;
    if (const char* env = getenv("HOLO_ATTN_CTAS"))
        if (atoi(env) > 0) want = (uint64_t)atoi(env);
    const uint64_t total = (uint64_t)tiles_per_plane * planes;
    return (uint32_t)(want < total ? want : total);
}

}  // namespace

int32_t holo_launch_decode_attention(holo_b200_ctx* ctx, const HoloAttnArgs& a) {
    const uint32_t G = a.h / a.hkv, planes = a.b * a.hkv;
    const bool aligned = (((uintptr_t)a.k_past | (uintptr_t)a.v_past | (uintptr_t)a.k_past_s | (uintptr_t)a.v_past_s |
                           (uintptr_t)a.k_new | (uintptr_t)a.v_new) & 15u) == 0;
    const bool tiled = !a.mask && a.quantized && a.d == HD && a.m == 1 && a.nnew == 1 && G <= MAXG && a.past >= 4 && (a.past % 4) == 0 &&
                       aligned && planes <= 65535 && encode_tiled_fn() != nullptr && !getenv("HOLO_ATTN_FORCE_GENERIC");
    if (!tiled) {
        if (a.d > 32 * holo_attn::GEN_MAX_PER_LANE)
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode attention head_dim %u exceeds %d", a.d, 32 * holo_attn::GEN_MAX_PER_LANE);
        const uint64_t rows = (uint64_t)a.b * a.h * a.m;
        if (rows > 0x7fffffffull) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode attention row count too large");
        const size_t smem = (size_t)holo_attn::GEN_WARPS * (a.d + 2) * sizeof(float);
        if (a.quantized)
            HOLO_CUDA(holo_launch_kernel(ctx, holo_attn::decode_attention_generic_kernel<true>, dim3((unsigned)rows), dim3(holo_attn::GEN_WARPS * 32), smem, 1, a));
        else
            HOLO_CUDA(holo_launch_kernel(ctx, holo_attn::decode_attention_generic_kernel<false>, dim3((unsigned)rows), dim3(holo_attn::GEN_WARPS * 32), smem, 1, a));
        HOLO_CUDA(cudaGetLastError());
        ctx->launches++;
        return HOLO_OK;
    }
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        HOLO_CUDA(cudaFuncSetAttribute(decode_attention_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        configured_device = ctx->device;
    }
    const uint32_t tiles = (a.past + TK - 1) / TK + 1;
    const uint32_t nctas = persistent_ctas(tiles, planes, ctx->sm_count);
    const uint32_t max_slots = nctas / planes + 2;
    const uint32_t box_rows = a.past < (uint32_t)TK ? a.past : (uint32_t)TK;
    const uint64_t po_bytes = (uint64_t)planes * max_slots * MAXG * HD * 4, pml_bytes = (uint64_t)planes * max_slots * MAXG * 2 * 4;
    HOLO_TRY(holo_ensure_scratch(ctx, po_bytes + pml_bytes));
    CUtensorMap mk, mv, mks, mvs;
    HOLO_TRY(make_codes_map(&mk, a.k_past, a.past, planes, box_rows));
    HOLO_TRY(make_codes_map(&mv, a.v_past, a.past, planes, box_rows));
    HOLO_TRY(make_scales_map(&mks, a.k_past_s, a.past, planes, box_rows));
    HOLO_TRY(make_scales_map(&mvs, a.v_past_s, a.past, planes, box_rows));
    FaParams p;
    p.q = a.q;
    p.k_new = (const int8_t*)a.k_new;
    p.v_new = (const int8_t*)a.v_new;
    p.k_new_s = a.k_new_s;
    p.v_new_s = a.v_new_s;
    p.valid_len = a.valid_len;
    p.out = a.out;
    p.part_o = (float*)ctx->scratch;
    p.part_ml = (float*)((uint8_t*)ctx->scratch + po_bytes);
    p.status = ctx->dev_status;
    p.arrivals = ctx->attn_arrivals;
    p.past = a.past;
    p.G = G;
    p.planes = planes;
    p.max_slots = max_slots;
    p.box_rows = box_rows;
    p.scale_div = a.scale_div;
    p.dtype = a.dtype;
    HOLO_CUDA(holo_launch_kernel(ctx, decode_attention_q8_kernel, dim3(nctas), dim3(FA_THREADS), SMEM_TOTAL, 1, mk, mv, mks, mvs, p));
    HOLO_CUDA(cudaGetLastError());
    ctx->launches++;
    return HOLO_OK;
}

// ---- allocation-free entry point ----------------------------------------------------------------
// Some callers must not allocate device memory when they run attention: a serving loop that
// has handed all of HBM to its own arena and treats any cudaMalloc as a fault, or code running
// where the CUDA allocator may synchronise the device and stall every other stream. For them
// the split-KV partials live in a fixed array that is part of the library image instead of the
// context's growable scratch buffer. Every GPU that loads the library holds these 16 MiB until
// the process exits.
constexpr uint64_t STATIC_SCRATCH_BYTES = 16ull << 20;
static __device__ __align__(256) unsigned char g_attn_static_scratch[STATIC_SCRATCH_BYTES];
// word 0: status; words 64..: one arrival counter per plane (at most 65535 planes)
static __device__ __align__(256) uint32_t g_attn_static_status[64 + 65536];

namespace {
struct StaticDevice {
    void* scratch = nullptr;
    uint32_t* status = nullptr;
    int sm_count = 0;
    bool ready = false;
};
StaticDevice g_static_dev[64];
std::mutex g_static_mutex;   // the first call on a device may come from several host threads at once

// One-time set-up for the calling thread's current device. In host code the arrays' names are only
// handles for the runtime: the addresses a kernel can use come from cudaGetSymbolAddress, with
// this device current.
int32_t static_device(StaticDevice** out) {
    int dev = 0;
    HOLO_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticDevice& sd = g_static_dev[dev];
    if (!sd.ready) {
        HOLO_CUDA(cudaGetSymbolAddress(&sd.scratch, g_attn_static_scratch));
        HOLO_CUDA(cudaGetSymbolAddress((void**)&sd.status, g_attn_static_status));
        HOLO_CUDA(cudaDeviceGetAttribute(&sd.sm_count, cudaDevAttrMultiProcessorCount, dev));
        HOLO_CUDA(cudaFuncSetAttribute(decode_attention_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        sd.ready = true;
    }
    *out = &sd;
    return HOLO_OK;
}
}  // namespace

extern "C" int32_t holo_b200_decode_attention_q8_static(void* cuda_stream, const void* q, const int8_t* k_past,
                                                        const float* k_past_scales, const int8_t* v_past,
                                                        const float* v_past_scales, const int8_t* k_new,
                                                        const float* k_new_scales, const int8_t* v_new,
                                                        const float* v_new_scales, const uint32_t* valid_len, void* out,
                                                        uint32_t batch, uint32_t heads, uint32_t kv_heads, uint32_t past_len,
                                                        uint32_t head_dim, uint32_t scale_bits, uint8_t dtype) {
    if (batch == 0 || heads == 0 || head_dim == 0) return HOLO_OK;
    const uint32_t hkv = kv_heads == 0 ? heads : kv_heads;
    if (hkv == 0 || heads % hkv != 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode_attention_valid: heads must be a multiple of kv_heads (grouped-query)");
    if (!holo_is_compute_float(dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode_attention_q8_static: q/output dtype must be f32, f16 or bf16");
    const uint32_t G = heads / hkv, planes = batch * hkv;
    const bool aligned = (((uintptr_t)k_past | (uintptr_t)v_past | (uintptr_t)k_past_scales | (uintptr_t)v_past_scales |
                           (uintptr_t)k_new | (uintptr_t)v_new) & 15u) == 0 &&
                         (((uintptr_t)valid_len | (uintptr_t)k_new_scales | (uintptr_t)v_new_scales) & 3u) == 0;
    if (head_dim != HD || G > MAXG || past_len < 4 || (past_len % 4) != 0 || !aligned || planes > 65535 || encode_tiled_fn() == nullptr)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP,
                         "unsupported op: decode_attention_q8_static serves head_dim 128, at most 4 query heads per kv head, a cache "
                         "bucket that is a multiple of 4 rows, 16-byte aligned code/scale pointers and batch*kv_heads <= 65535");
    StaticDevice* sdp = nullptr;
    HOLO_TRY(static_device(&sdp));   // the first call on a device sets it up: make it before any stream capture
    StaticDevice& sd = *sdp;
    const uint32_t tiles = (past_len + TK - 1) / TK + 1;
    const uint32_t nctas = persistent_ctas(tiles, planes, sd.sm_count);
    const uint32_t max_slots = nctas / planes + 2;
    const uint64_t po_bytes = (uint64_t)planes * max_slots * MAXG * HD * 4, pml_bytes = (uint64_t)planes * max_slots * MAXG * 2 * 4;
    if (po_bytes + pml_bytes > STATIC_SCRATCH_BYTES)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP,
                         "unsupported op: decode_attention_q8_static needs %llu bytes of split-KV partials for this shape; the built-in "
                         "scratch holds %llu (use holo_b200_dispatch, whose scratch grows)",
                         (unsigned long long)(po_bytes + pml_bytes), (unsigned long long)STATIC_SCRATCH_BYTES);
    float scale_div = sqrtf((float)head_dim);
    if (scale_div < 1.0f) scale_div = 1.0f;
    if (scale_bits != 0) {
        float sm;
        memcpy(&sm, &scale_bits, 4);
        if (sm > 0.0f) scale_div = 1.0f / sm;
    }
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const uint32_t box_rows = past_len < (uint32_t)TK ? past_len : (uint32_t)TK;
    CUtensorMap mk, mv, mks, mvs;
    HOLO_TRY(make_codes_map(&mk, k_past, past_len, planes, box_rows));
    HOLO_TRY(make_codes_map(&mv, v_past, past_len, planes, box_rows));
    HOLO_TRY(make_scales_map(&mks, k_past_scales, past_len, planes, box_rows));
    HOLO_TRY(make_scales_map(&mvs, v_past_scales, past_len, planes, box_rows));
    // The planes' arrival counters must start at zero (a launch that gave up may have left counts
    // behind). The partials need no clearing: every (plane, slot) the merge reads is rewritten first.
    // The status word is NOT cleared here: a bounded wait that gave up stays recorded (and the CTAs of
    // later launches return at once, writing nothing) until holo_b200_decode_attention_q8_static_status
    // has reported it.
    HOLO_CUDA(cudaMemsetAsync(sd.status + 64, 0, (size_t)planes * sizeof(uint32_t), stream));
    FaParams p;
    p.q = q;
    p.k_new = k_new;
    p.v_new = v_new;
    p.k_new_s = k_new_scales;
    p.v_new_s = v_new_scales;
    p.valid_len = valid_len;
    p.out = out;
    p.part_o = (float*)sd.scratch;
    p.part_ml = (float*)((uint8_t*)sd.scratch + po_bytes);
    p.status = sd.status;
    p.arrivals = sd.status + 64;
    p.past = past_len;
    p.G = G;
    p.planes = planes;
    p.max_slots = max_slots;
    p.box_rows = box_rows;
    p.scale_div = scale_div;
    p.dtype = dtype;
    decode_attention_q8_kernel<<<nctas, FA_THREADS, SMEM_TOTAL, stream>>>(mk, mv, mks, mvs, p);
    HOLO_CUDA(cudaGetLastError());
    return HOLO_OK;
}

// Device-side failures of the allocation-free entry point. The launches above return before the
// kernel has run, so a bounded wait that gives up inside it (its CTAs then return without writing
// `out`) can only be reported afterwards: this call copies the 4-byte status word back on
// `cuda_stream` (a device-to-host copy of the built-in word: no allocation), waits for the stream,
// and returns HOLO_ERR_DISPATCH if a wait gave up since the last query, clearing the record so
// that later calls run again. HOLO_OK otherwise.
extern "C" int32_t holo_b200_decode_attention_q8_static_status(void* cuda_stream) {
    StaticDevice* sd = nullptr;
    HOLO_TRY(static_device(&sd));
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    uint32_t st = 0;
    HOLO_CUDA(cudaMemcpyAsync(&st, sd->status, 4, cudaMemcpyDeviceToHost, stream));
    HOLO_CUDA(cudaStreamSynchronize(stream));
    if (st == 0) return HOLO_OK;
    HOLO_CUDA(cudaMemsetAsync(sd->status, 0, 4, stream));
    return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: a device-side bounded wait gave up in decode_attention_q8_static (status 0x%x)", st);
}
