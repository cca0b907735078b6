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
//     While the ring is full the same warp prepares the query digits of the share's next plane
//     in a second digit tile, so the consumers change planes without rebuilding them.
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

#include <algorithm>
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
constexpr uint32_t SMEM_Q = STAGES * STAGE_BYTES;            // two 16 x 128 B query digit tiles (this segment's, the next one's)
constexpr uint32_t SMEM_MISC = SMEM_Q + 2 * 16 * HD;         // cq[2][4], bad[2][4], abort, barriers
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
    return exp2f(s - m);
}

// Digits of one query element against its head's exponent: qi = rn(q * 2^(21-ex)), |qi| < 2^22, cut into
// three signed base-256 digits (L0 most significant). The power of two is built from its bits where it is
// a normal number (exact, like scalbnf) and by scalbnf otherwise (heads whose largest element is below 2^-105).
__device__ __forceinline__ void q_digits(float qv, int ex, int& L0, int& L1, int& L2) {
    const float scaled = ex >= -105 ? qv * __uint_as_float((uint32_t)(127 + 21 - ex) << 23) : scalbnf(qv, 21 - ex);
    const int qi = __float2int_rn(scaled);
    L2 = ((qi + 128) & 255) - 128;
    const int q1 = (qi - L2) >> 8;
    L1 = ((q1 + 128) & 255) - 128;
    L0 = (q1 - L1) >> 8;
}
__device__ __forceinline__ float q_unit(int ex, float scale_div) {   // 2^(ex-21) / scale_div
    const float u = ex >= -105 ? __uint_as_float((uint32_t)(127 + ex - 21) << 23) : scalbnf(1.0f, ex - 21);
    return u / scale_div;
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
                    const float fo = exp2_guard(M[gg], nm), fn = exp2f(wm - nm);
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
// each segment the consumers take the query digits (built by themselves for the first segment, by
// the producer warp for the later ones), run the tiles, merge their four running
// (max, sum, context) triples, and either write the plane's result (the CTA had the whole plane)
// or store a partial and count in on the plane's arrival counter; the CTA that counts in last
// merges the plane's partials. Nobody waits for anybody: a CTA that is not last simply goes on.
__global__ void __launch_bounds__(FA_THREADS, HOLO_ATTN_MINB)
decode_attention_q8_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                           const __grid_constant__ CUtensorMap map_ks, const __grid_constant__ CUtensorMap map_vs,
                           const FaParams p) {
    holo_pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    float* s_cq = reinterpret_cast<float*>(sm + SMEM_MISC);            // [2][4]
    uint32_t* s_bad = reinterpret_cast<uint32_t*>(sm + SMEM_MISC + 64);  // [2][4]
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(sm + SMEM_MISC + 32);
    uint32_t* s_fast = reinterpret_cast<uint32_t*>(sm + SMEM_MISC + 36);
    uint32_t* s_last = reinterpret_cast<uint32_t*>(sm + SMEM_MISC + 192);  // [9]
    const uint32_t bar_full = base + SMEM_MISC + 128, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_q_full = base + SMEM_MISC + 96, bar_q_empty = bar_q_full + 16;   // two digit tiles: filled / read
    float* mo = reinterpret_cast<float*>(sm + SMEM_MERGE);  // [warp][head][HD]
    float* mml = mo + CONSUMER_WARPS * MAXG * HD;            // [warp][head][2]
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // what touches no global memory is done while the previous kernel drains
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, CONSUMER_WARPS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_q_full + 8 * b, 1);
            mbar_init(bar_q_empty + 8 * b, CONSUMER_WARPS);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    holo_pdl_wait();

    const uint32_t G = p.G, nctas = gridDim.x, cta = blockIdx.x;
    // an earlier launch gave up on a wait: do not start (both loads are in flight together)
    const uint32_t sticky = *reinterpret_cast<volatile uint32_t*>(p.status);
    const uint32_t vis_past = min(*p.valid_len, p.past);
    const uint32_t tiles_past = (vis_past + TK - 1) / TK;
    const uint32_t T = tiles_past + 1;  // + the tile holding this step's new row
    const uint32_t total = p.planes * T;
    const uint32_t g0 = fa_start(cta, total, nctas), g1 = fa_start(cta + 1, total, nctas);
    if (sticky & 2u) return;
    __syncthreads();

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer warp ----------------
        const uint32_t tx_bytes = p.box_rows * HD * 2 + p.box_rows * 4 * 2;
        // Besides feeding the ring, this warp prepares the query digits of every segment of the share (one
        // segment = the share's tiles of one plane) in its idle time, one segment ahead of the consumers:
        // q = (L0*65536 + L1*256 + L2) * 2^(ex-21) per head, one row of the m16 tile per (head, digit): rows g,
        // 4+g, 8+g hold L0, L1, L2 of head g; rows 12.. are zero. Two digit tiles alternate; a tile is
        // rewritten only after all four consumer warps have taken the previous content into registers.
        const uint32_t plane0 = g0 / T;
        const uint32_t nseg = g1 > g0 ? (g1 - 1) / T - plane0 + 1 : 0;
        // the first segment's digits are made by the consumer warps themselves (they have nothing else to do yet)
        uint32_t job = 1, job_head = 0;   // segment whose digits come next; heads of it already written
        bool dead = false;
        // the job's query elements (this lane's four per head): requested when the job before it is finished
        // (the first job's before the first tiles), so a whole segment lies between the request and the use
        float qj[MAXG][4];
        auto job_load = [&]() {
#pragma unroll
            for (int h = 0; h < MAXG; ++h)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    qj[h][e] = (job < nseg && (uint32_t)h < G) ? holo::load_float(p.q, ((uint64_t)(plane0 + job) * G + h) * HD + 4 * lane + e, p.dtype) : 0.0f;
        };
        job_load();
        auto job_step = [&]() {           // one head of segment `job`; whole warp
            const uint32_t b = job & 1u, gg = job_head;
            if (gg == 0 && job >= 2) {
                bool ok = true;
                if (lane == 0) ok = mbar_wait(bar_q_empty + 8 * b, ((job >> 1) - 1) & 1, s_abort, p.status);
                if (!__shfl_sync(0xffffffffu, ok, 0)) { dead = true; return; }
            }
            float qv[4];
            float a = 0.0f;
            bool isnan_ = false;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                qv[e] = gg == 0 ? qj[0][e] : gg == 1 ? qj[1][e] : gg == 2 ? qj[2][e] : qj[3][e];
                a = fmaxf(a, fabsf(qv[e]));
                isnan_ |= qv[e] != qv[e];   // NaN elements are dropped by fmaxf; detect them separately
            }
            for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            const float amax = __any_sync(0xffffffffu, isnan_) ? INFINITY : a;
            const uint32_t be = (__float_as_uint(amax) >> 23) & 0xffu;
            uint32_t w0 = 0, w1 = 0, w2 = 0, bad = 0;
            float cqv = 0.0f;
            if (be == 255u) {
                bad = 1;  // inf / NaN in q: the reference yields NaN for the whole head
            } else if (be != 0u) {
                const int ex = (int)be - 127;  // amax < 2^(ex+1)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int L0, L1, L2;
                    q_digits(qv[e], ex, L0, L1, L2);
                    w0 |= ((uint32_t)L0 & 0xffu) << (8 * e);
                    w1 |= ((uint32_t)L1 & 0xffu) << (8 * e);
                    w2 |= ((uint32_t)L2 & 0xffu) << (8 * e);
                }
                cqv = q_unit(ex, p.scale_div);
            }
            uint32_t* sq32 = reinterpret_cast<uint32_t*>(sm + SMEM_Q + b * 16 * HD);
            sq32[(gg * HD) / 4 + lane] = w0;
            sq32[((4 + gg) * HD) / 4 + lane] = w1;
            sq32[((8 + gg) * HD) / 4 + lane] = w2;
            sq32[((12 + gg) * HD) / 4 + lane] = 0;
            if (lane == 0) {
                s_cq[b * 4 + gg] = cqv;
                s_bad[b * 4 + gg] = bad;
            }
            if (++job_head == (uint32_t)MAXG) {
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_q_full + 8 * b);
                job_head = 0;
                ++job;
                job_load();
            }
        };
        asm volatile("bar.sync 2, %0;" ::"n"(FA_THREADS) : "memory");   // the consumers' first query loads are out
        uint32_t it = 0;
        for (uint32_t g = g0; g < g1 && !dead; ++g, ++it) {
            const uint32_t s = it % STAGES, use = it / STAGES;
            const uint32_t plane = g / T, t = g % T;
            const uint32_t seg = plane - plane0;
            // the first round of tiles goes out before anything else; from then on a segment's digits are complete
            // before its first tile is handed over, and the next segment's are worked on while the ring is full
            if (use > 0 || g + 1 == g1) {
                while (job <= seg && !dead) job_step();
            }
            if (use > 0) {
                while (job < nseg && job <= seg + 1 && !dead) {
                    uint32_t free_now = 0;
                    if (lane == 0) free_now = mbar_try_wait(bar_empty + 8 * s, (use - 1) & 1);
                    if (__shfl_sync(0xffffffffu, free_now, 0)) break;
                    job_step();
                }
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
        while (job < nseg && !dead) job_step();
        return;
    }

    // ---------------- consumer warps ----------------
    const uint32_t r = lane >> 2, i = lane & 3;
    const bool hi_group = r >= 4;       // lanes holding digit L1 (and the zero row)
    const uint32_t g = r & 3;           // head served by this lane
    const uint32_t selA = hi_group ? 0x0051u : 0x0062u;  // digit byte of (x, y): L1 = byte 1, L0 = byte 2
    const uint32_t selB = hi_group ? 0x0073u : 0x0040u;  // zero byte 3, or L2 = byte 0
    const float digit_w = hi_group ? 256.0f : 65536.0f;  // weight of the group's first digit row against its second
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
    // thread 0: a partial that has been stored but not yet counted in on its plane (see below)
    bool pub_wait = false;
    uint32_t pub_plane = 0, pub_first = 0, pub_last = 0, pub_sharers = 0;
    auto count_in = [&]() {
        __threadfence();   // release: the CTA's stores were ordered before this thread by the barrier after them
        if (npend < 2) {
            // the count comes back while the next segment streams; it is read at the end
            pend_before[npend] = atomicAdd(p.arrivals + pub_plane, 1u);
            pend_plane[npend] = pub_plane;
            pend_first[npend] = pub_first;
            pend_last[npend] = pub_last;
            pend_sharers[npend] = pub_sharers;
            ++npend;
        }
        pub_wait = false;
    };
    uint32_t seg_no = 0, bad_heads = 0;
    // The first plane's query is requested before the producer asks for its first tiles: behind those 100 KB per
    // CTA the few hundred bytes would wait for microseconds.
    float q_first[MAXG];
#pragma unroll
    for (int gg = 0; gg < MAXG; ++gg)
        q_first[gg] = (g0 < g1 && (uint32_t)gg < G) ? holo::load_float(p.q, ((uint64_t)(g0 / T) * G + gg) * HD + tid, p.dtype) : 0.0f;
    asm volatile("bar.arrive 2, %0;" ::"n"(FA_THREADS) : "memory");
    while (gt < g1) {
        const uint32_t plane = gt / T;
        const uint32_t seg_end = min(g1, (plane + 1) * T);
        // the plane's first sharer looks at the arrival counter now and uses the value when the
        // segment ends, so the round trip is hidden behind the segment's tiles
        uint32_t probe = 0;
        if (tid == 0 && fa_owner(plane * T, total, nctas) == cta && fa_owner(plane * T + T - 1, total, nctas) != cta)
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(probe) : "l"(p.arrivals + plane) : "memory");
        // ---- query digits of this plane, prepared by the producer warp: A fragments, scale, bad-head flags ----
        {
            const uint32_t qb = seg_no & 1u;
            if (seg_no == 0) {
                // the share's first plane: all four warps build the digit tile (thread = element of the head)
                int8_t* sq = reinterpret_cast<int8_t*>(sm + SMEM_Q);
                float* s_red = mo;   // the merge area is idle until the segment ends
                float qv[MAXG];
#pragma unroll
                for (int gg = 0; gg < MAXG; ++gg) {
                    qv[gg] = q_first[gg];
                    float a = fabsf(qv[gg]);
                    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
                    const uint32_t nanbit = __any_sync(0xffffffffu, qv[gg] != qv[gg]);
                    if (lane == 0) s_red[warp * 4 + gg] = nanbit ? INFINITY : a;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
                for (int gg = 0; gg < MAXG; ++gg) {
                    const float amax = fmaxf(fmaxf(s_red[gg], s_red[4 + gg]), fmaxf(s_red[8 + gg], s_red[12 + gg]));
                    const uint32_t be = (__float_as_uint(amax) >> 23) & 0xffu;
                    int L0 = 0, L1 = 0, L2 = 0;
                    if (be != 255u && be != 0u) q_digits(qv[gg], (int)be - 127, L0, L1, L2);
                    sq[gg * HD + tid] = (int8_t)L0;
                    sq[(4 + gg) * HD + tid] = (int8_t)L1;
                    sq[(8 + gg) * HD + tid] = (int8_t)L2;
                    sq[(12 + gg) * HD + tid] = 0;
                    if (tid == 0) {
                        s_cq[gg] = (be != 255u && be != 0u) ? q_unit((int)be - 127, p.scale_div) : 0.0f;
                        s_bad[gg] = be == 255u;   // inf / NaN in q: the reference yields NaN for the whole head
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (tid == 0) mbar_arrive(bar_q_full);   // keeps the tile's phases in step with the producer's
            } else if (!aborted && !mbar_wait(bar_q_full + 8 * qb, (seg_no >> 1) & 1, s_abort, p.status)) {
                aborted = true;
            }
            cq = s_cq[qb * 4 + g] * LOG2E;   // scores, running maxima and the stored partial maxima are in log2 units
            bad_heads = s_bad[qb * 4] | (s_bad[qb * 4 + 1] << 1) | (s_bad[qb * 4 + 2] << 2) | (s_bad[qb * 4 + 3] << 3);
            const uint32_t* sq32 = reinterpret_cast<const uint32_t*>(sm + SMEM_Q + qb * 16 * HD);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                qa[ks][0] = sq32[(r * HD + 32 * ks + 4 * i) >> 2];
                qa[ks][1] = sq32[((r + 8) * HD + 32 * ks + 4 * i) >> 2];
                qa[ks][2] = sq32[(r * HD + 32 * ks + 16 + 4 * i) >> 2];
                qa[ks][3] = sq32[((r + 8) * HD + 32 * ks + 16 + 4 * i) >> 2];
            }
            __syncwarp();
            if (lane == 0 && !aborted) mbar_arrive(bar_q_empty + 8 * qb);   // the tile may be rewritten
            ++seg_no;
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
                // Both lane groups hold digit sums of the same 8 (head, key) scores (the low group L0 and L2, the
                // high group L1). Each group finishes four of them: the low group those of key blocks 0 and 1, the
                // high group those of blocks 2 and 3; it gets the partner's part of its own four by one shuffle
                // each and hands the finished weights back the same way. Everything in between (scales, exp,
                // digit scaling) then runs once per score instead of once per group.
                float sc[4], svv[4];
                float mt = -INFINITY;
    #pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    const int nt_lo = h2, nt_hi = 2 + h2;
                    const uint32_t key = row0 + 8 * (hi_group ? nt_hi : nt_lo) + 2 * i;
                    const float2 k2 = *reinterpret_cast<const float2*>(sk + key);
                    const float2 v2 = *reinterpret_cast<const float2*>(sv + key);
    #pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        // this lane's digits of the low group's score and of the high group's score (the high group's
                        // second row is the zero row, so one formula with the group's digit weight serves both)
                        const float for_lo = fmaf(__int2float_rn(sacc[nt_lo][e]), digit_w, __int2float_rn(sacc[nt_lo][2 + e]));
                        const float for_hi = fmaf(__int2float_rn(sacc[nt_hi][e]), digit_w, __int2float_rn(sacc[nt_hi][2 + e]));
                        const float theirs = __shfl_xor_sync(0xffffffffu, hi_group ? for_lo : for_hi, 16);
                        const float full = (hi_group ? for_hi : for_lo) + theirs;
                        float kscale = e ? k2.y : k2.x;
                        float sval = full * (kscale * cq);
                        float vscale = e ? v2.y : v2.x;
                        if (key + e >= limit) {  // unrealized row: whatever bytes it holds never count
                            sval = -INFINITY;
                            vscale = 0.0f;
                        }
                        sc[h2 * 2 + e] = sval;
                        svv[h2 * 2 + e] = vscale;
                        mt = fmaxf(mt, sval);
                    }
                }
                // ---- weights relative to the running reference, scaled for digit extraction ----
                float pe[4], ps[4];
                // largest scaled weight, compared as bit patterns: for weights >= 0 that is the float order, and a NaN
                // or a negative value (a corrupt scale) compares above every finite weight, which forces the fold
                uint32_t pmax = 0u;
    #pragma unroll
                for (int x = 0; x < 4; ++x) {
                    // before the first fold m_ref is -inf and sref 0: whatever comes out here is recomputed below
                    pe[x] = exp2f(sc[x] - m_ref);
                    ps[x] = pe[x] * svv[x] * sref;
                    pmax = max(pmax, __float_as_uint(ps[x]));
                }
                // each lane judges its own four scores; the maxima over a head's lanes are only formed when some lane
                // of the warp asks for a new reference (rare), which keeps six dependent shuffles off every tile
                const bool need = !(pmax < 0x4B7FFFFFu) || mt > m_ref + 86.0f || sref == 0.0f || since_fold >= 1024;
                if (__any_sync(0xffffffffu, need)) {
                    fold();
                    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
                    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
                    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
                    const float m_new = fmaxf(m_ref, mt);
                    const float alpha = m_ref == -INFINITY ? 0.0f : exp2f(m_ref - m_new);
    #pragma unroll
                    for (int x = 0; x < 32; ++x) of[x] *= alpha;
                    l_sum *= alpha;
                    m_ref = m_new;
                    float pm = 0.0f;
    #pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        pe[x] = exp2_guard(sc[x], m_ref);
                        float w = pe[x] * svv[x];
                        pm = fmaxf(pm, w);
                    }
                    pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 1));
                    pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 2));
                    pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 16));
                    int sexp = 0;
                    const uint32_t pbe = (__float_as_uint(pm) >> 23) & 0xffu;
                    if (pbe != 0u && pbe != 255u) sexp = 15 - ((int)pbe - 127);
                    sexp = max(-100, min(100, sexp));
                    sref = __uint_as_float((uint32_t)(127 + sexp) << 23);
                    inv_sref = __uint_as_float((uint32_t)(127 - sexp) << 23);
    #pragma unroll
                    for (int x = 0; x < 4; ++x) ps[x] = fminf(pe[x] * svv[x] * sref, 16777215.0f);
                }
                uint32_t pi[8];
    #pragma unroll
                for (int x = 0; x < 4; ++x) {
                    l_sum += pe[x];   // this group's four keys; the groups' sums meet when the segment ends
                    const uint32_t mine = __float2uint_rn(ps[x]);   // saturating: a negative or NaN weight (a corrupt scale) counts as 0
                    const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, 16);
                    pi[x] = hi_group ? theirs : mine;
                    pi[4 + x] = hi_group ? mine : theirs;
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
            if (tid == 0 && pub_wait) count_in();
        }
        fold();
        // ---- merge the four warps' triples; finish the plane or publish this segment's partial ----
        l_sum += __shfl_xor_sync(0xffffffffu, l_sum, 1);
        l_sum += __shfl_xor_sync(0xffffffffu, l_sum, 2);
        l_sum += __shfl_xor_sync(0xffffffffu, l_sum, 16);
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
                            float f = exp2f(wm - M[gg]);
                            L[gg] = fmaf(mml[(w * MAXG + gg) * 2 + 1], f, L[gg]);
                            O[gg] = fmaf(mo[(w * MAXG + gg) * HD + c], f, O[gg]);
                        }
                    }
                    if ((bad_heads >> gg) & 1u) { O[gg] = NAN; L[gg] = 1.0f; M[gg] = 0.0f; }
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
                // Counting in needs the partial to be visible first. The barrier that ends the segment orders every
                // thread's stores before thread 0; thread 0 then fences and counts in after the next segment's first
                // tile (or before the final merges), when the stores have long drained and the fence costs nothing.
                if (tid == 0) {
                    pub_wait = true;
                    pub_plane = plane;
                    pub_first = first;
                    pub_last = last;
                    pub_sharers = sharers;
                }
            }
        }
        // the merge area is rewritten by the next segment
        asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    // ---- a CTA that counted in last on a plane merges that plane's partials ----
    if (tid == 0 && pub_wait) count_in();
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

// Grid of the persistent kernel: at most HOLO_ATTN_MINB CTAs per SM (all co-resident), never more than
// there are tiles. Shares that line up with the planes are worth a few idle CTA slots: a CTA that holds
// whole planes neither stores partials nor merges, and one that holds an exact fraction of a plane never
// changes planes in mid-share. So when the plane count divides evenly into at least three quarters of the
// slots (k CTAs per plane, or m planes per CTA), that count is taken; measured on B200 at 256 of 296 slots:
// 101.7 -> 91.6 us for 256 planes x 65 tiles, 59.8 -> 51.7 us for 128 planes x 33 tiles. Otherwise every slot
// is used and a plane is shared by at most nctas / planes + 2 CTAs.
uint32_t persistent_ctas(uint32_t tiles_per_plane, uint32_t planes, int sm_count) {
    uint64_t slots = (uint64_t)HOLO_ATTN_MINB * (uint32_t)sm_count;
    const uint64_t total = (uint64_t)tiles_per_plane * planes;
    if (const char* env = getenv("HOLO_ATTN_CTAS"))
        if (atoi(env) > 0) return (uint32_t)std::min<uint64_t>((uint64_t)atoi(env), total);
    uint64_t want = slots;
    if (planes > 0 && planes <= slots) {
        const uint64_t k = slots / planes;
        if (planes * k * 4 >= slots * 3 && k <= tiles_per_plane) want = planes * k;
    } else if (planes > slots) {
        const uint64_t m = (planes + slots - 1) / slots;
        if (planes % m == 0 && (planes / m) * 4 >= slots * 3) want = planes / m;
    }
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
