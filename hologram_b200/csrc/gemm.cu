// bf16 matmul with f32 accumulation and bf16 (truncated) output, plus the fused epilogues.
// Replaces matmul_float / matmul_activation_float / matmul_add_float
// (crates/hologram-compute/src/cpu/float_kernels.rs:298-399, 822-891): C = trunc_bf16(A[m,k] . B[k,n]),
// both operands row-major; the epilogue re-widens the truncated product, applies the
// activation (as a lookup in the 16-bit LUT, bit-identical to the CPU's scalar function) or
// adds the residual in f32, and truncates again.
//
// Tensor-core kernel (sm_100a): one 128 x BN output tile per CTA, K in 64-wide blocks.
//   warp 0   TMA producer: A tile (K-major, 128B swizzle) and B tile (N-major, 128B swizzle)
//            into a shared-memory ring, mbarrier full/empty pairs
//   warp 1   tcgen05.mma issuer (one elected lane), accumulator in TMEM (128 lanes x BN columns);
//            tcgen05.commit releases ring slots and signals the epilogue
//   warps 2-5 epilogue: tcgen05.ld the accumulator rows, narrow, epilogue op, store
// Skinny problems (few output tiles) split K across the CTAs of a thread-block cluster (up to 8
// along grid z): every CTA parks its f32 accumulator tile in its own shared memory, and after a
// cluster barrier CTA r sums rows r, r + S, ... of the tile over all S CTAs through distributed
// shared memory, in split order, and applies the epilogue (one truncation, as the reference).
// No partial ever goes to global memory and there is no second launch. Every mbarrier wait is bounded; a wait that gives up raises a status bit, and
// the CTA still frees its TMEM before it exits.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.h"
#include "numerics.cuh"
#include "p2p.cuh"

namespace {

constexpr int BM = 128, BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 20;

// One output segment: columns [col_begin, col_end) of the product go to their own row-major
// [m, col_end - col_begin] buffer with their own epilogue. A plain matmul has one segment; the
// session's sibling-matmul merge (several products of the same A against concatenated weights)
// has up to three. Segment boundaries are multiples of 32 columns.
struct GemmSeg {
    uint16_t* out;            // bf16 output
    const uint16_t* table;    // 65536-entry LUT of the fused activation or null
    const uint16_t* residual; // bf16 [m, width] or null
    uint32_t col_begin, col_end;
    // per-head work on the stored values (heads of 128 columns, one tile each; see HoloMatmulSeg::head_op)
    uint32_t head_op;
    const uint16_t *cos, *sin;
    uint16_t* rope_out;
    int8_t* codes;
    float* scales;
};
constexpr int MAX_SEGS = 3;

struct GemmParams {
    GemmSeg seg[MAX_SEGS];
    uint32_t nseg;
    uint32_t* status;
    uint32_t m, n, k, kblocks, splits, box_m;
    int dtype;                // HOLO_DTYPE_BF16 or HOLO_DTYPE_F16 (operands and output)
    uint32_t gated;           // see HoloMatmulSeg::gated (BN = 128: columns 0..63 of a tile are gate, 64..127 up)
    uint32_t head_ops;        // some segment has a head_op (BN = 128, K split inside a cluster)
    uint32_t b_constant;      // B is a weight no kernel of the stream writes: its first tiles may be requested before the dependency wait
    // tensor-parallel sum inside the epilogue (ar_world > 1): every rank's mailbox, the local epoch /
    // ticket words, this rank
    uint8_t* ar_mailbox[8];
    uint32_t* ar_state;
    uint32_t ar_world, ar_rank;
    // CTA-pair kernel: work items [0, tail_begin) are whole 256 x 256 tiles; from tail_begin on every tile is two
    // items of 256 x 128 (the last, partial round of tiles is cut in two so that it keeps every pair busy)
    uint32_t tail_begin, n_items;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status) {
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (it > 64) __nanosleep(64);
    }
    *abort_flag = 1;
    atomicOr(status, 4u);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// Shared-memory matrix descriptor for tcgen05.mma: start address, leading / stride byte
// offsets (all in 16-byte units), descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// One 16-bit result: narrow the accumulator (bf16: truncation; f16: the reference's
// add-half rounding), then the fused epilogue on the narrowed value
// (float_kernels.rs:844-847, 886-889).
template <bool F16>
__device__ __forceinline__ uint16_t epilogue_elem(float acc, const uint16_t* table, const uint16_t* residual, uint64_t idx) {
    // the dtype is a compile-time choice: a run-time test per element made the bf16 epilogue of the
    // 4096^3 product a third slower
    constexpr int dtype = F16 ? HOLO_DTYPE_F16 : HOLO_DTYPE_BF16;
    uint16_t h = holo::narrow16(acc, dtype);
    if (table) h = __ldg(table + h);
    if (residual) h = holo::narrow16(__fadd_rn(holo::widen16(h, dtype), holo::widen16(__ldg(residual + idx), dtype)), dtype);
    return h;
}

// Gated pair: act(narrow(gate)) * narrow(up), both factors narrowed first, as the unfused
// MatMulActivation and MatMul would have stored them, the product narrowed once (binary Mul).
template <bool F16>
__device__ __forceinline__ uint16_t gated_elem(float gate, float up, const uint16_t* table) {
    constexpr int dtype = F16 ? HOLO_DTYPE_F16 : HOLO_DTYPE_BF16;
    uint16_t g = holo::narrow16(gate, dtype);
    if (table) g = __ldg(table + g);
    const uint16_t u = holo::narrow16(up, dtype);
    return holo::narrow16(__fmul_rn(holo::widen16(g, dtype), holo::widen16(u, dtype)), dtype);
}

// Tensor-parallel exchange of one unit (four narrowed results of this rank): `push` sends it to every
// peer's mailbox; `sum` polls the peers' units and returns the f32 sums in rank order (this rank's
// own value taking its place in the order). Same mailbox regions and epochs as the one-shot
// all-reduce kernel.
template <bool F16>
__device__ __forceinline__ uint2 ar_pack(const float (&a)[4]) {
    constexpr int dtype = F16 ? HOLO_DTYPE_F16 : HOLO_DTYPE_BF16;
    return make_uint2((uint32_t)holo::narrow16(a[0], dtype) | ((uint32_t)holo::narrow16(a[1], dtype) << 16),
                      (uint32_t)holo::narrow16(a[2], dtype) | ((uint32_t)holo::narrow16(a[3], dtype) << 16));
}
__device__ __forceinline__ void ar_push(const GemmParams& p, uint32_t epoch, uint64_t units, uint64_t unit, uint2 mine) {
    const uint64_t off = p2p_oneshot_offset(epoch);
    for (uint32_t k = 1; k < p.ar_world; ++k)
        ll_store(p.ar_mailbox[(p.ar_rank + k) % p.ar_world] + off, (uint64_t)p.ar_rank * units + unit, mine, epoch);
}
template <bool F16>
__device__ __forceinline__ bool ar_sum(const GemmParams& p, uint32_t epoch, uint64_t units, uint64_t unit, uint2 mine, float (&a)[4]) {
    constexpr int dtype = F16 ? HOLO_DTYPE_F16 : HOLO_DTYPE_BF16;
    const uint8_t* box = p.ar_mailbox[p.ar_rank] + p2p_oneshot_offset(epoch);
    a[0] = a[1] = a[2] = a[3] = 0.0f;
    for (uint32_t r = 0; r < p.ar_world; ++r) {
        uint2 v = mine;
        if (r != p.ar_rank && !ll_load(box, (uint64_t)r * units + unit, epoch, &v)) return false;
        a[0] = __fadd_rn(a[0], holo::widen16((uint16_t)(v.x & 0xffffu), dtype));
        a[1] = __fadd_rn(a[1], holo::widen16((uint16_t)(v.x >> 16), dtype));
        a[2] = __fadd_rn(a[2], holo::widen16((uint16_t)(v.y & 0xffffu), dtype));
        a[3] = __fadd_rn(a[3], holo::widen16((uint16_t)(v.y >> 16), dtype));
    }
    return true;
}

// A_ROWS = rows of the A tile that are backed by the ring (the TMA box never has more rows than
// min(m, 128)). With fewer than 128 the MMA still reads 128 rows: the rest is whatever follows in
// shared memory, and those accumulator rows are never stored. A smaller A slot buys more stages,
// i.e. more weight bytes in flight per CTA, which is what an HBM-bound skinny product needs.
template <int BN, int STAGES, int A_ROWS>
struct GemmSmem {
    static constexpr uint32_t A_BYTES = A_ROWS * BK * 2;       // 2, 8 or 16 KiB
    static constexpr uint32_t B_BYTES = BK * BN * 2;           // 8 or 16 KiB
    static constexpr uint32_t STAGE = A_BYTES + B_BYTES;
    static constexpr uint32_t RING = STAGES * STAGE + (BM - A_ROWS) * BK * 2;  // tail pad: the last A read stays in bounds
    static constexpr uint32_t BARS = (RING + 1023u) & ~1023u;   // full[STAGES], empty[STAGES], accum, tmem slot, abort, flag
    static constexpr uint32_t TOTAL = BARS + 256 + 1024;
};

// AR: the instantiation whose epilogue carries the tensor-parallel sum; the plain one compiles none of it
// (a run-time test in the epilogue cost the 4096^3 product a tenth of its time).
template <int BN, int STAGES, int A_ROWS, bool F16, bool AR>
__global__ void __launch_bounds__(GEMM_THREADS)
matmul_bf16_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using S = GemmSmem<BN, STAGES, A_ROWS>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    const uint32_t bar_full = base + S::BARS, bar_empty = bar_full + 8 * STAGES, bar_accum = bar_empty + 8 * STAGES;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(sm + S::BARS + 16 * STAGES + 8);
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(sm + S::BARS + 16 * STAGES + 12);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.x * BN, m0 = blockIdx.y * BM, split = blockIdx.z;
    const uint32_t kb_begin = (uint32_t)(((uint64_t)p.kblocks * split) / p.splits);
    const uint32_t kb_end = (uint32_t)(((uint64_t)p.kblocks * (split + 1)) / p.splits);
    const uint32_t nkb = kb_end - kb_begin;

    holo_pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_accum, 1);
        *s_abort = 0;   // the sticky abort bit of the status word is read by an epilogue warp, off the producer's path
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // TMEM accumulator: BN columns (power of two >= 32) x 128 lanes of f32
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *s_tmem;
    // A constant B (a weight nothing in the stream rewrites) does not depend on the previous kernel: the first
    // ring-full of its tiles is requested before the wait, so those bytes are on their way (or already here)
    // when A becomes readable. Each stage's barrier expects the A bytes too and completes only with them.
    const uint32_t pre = p.b_constant ? min(nkb, (uint32_t)STAGES) : 0u;
    if (warp == 0 && lane == 0) {
        const uint32_t tx = p.box_m * BK * 2 + S::B_BYTES;
        for (uint32_t i = 0; i < pre; ++i) {
            const uint32_t st = base + i * S::STAGE;
            const int k0 = (int)((kb_begin + i) * BK);
            mbar_arrive_expect_tx(bar_full + 8 * i, tx);
#pragma unroll
            for (int h = 0; h < BN / 64; ++h)
                tma_load_2d(st + S::A_BYTES + h * (BK * 128), &map_b, (int)(n0 + 64 * h), k0, bar_full + 8 * i);
        }
    }
    holo_pdl_wait();  // barriers and TMEM were set up while the previous kernel drained
    const uint32_t ar_epoch = (AR && p.ar_world > 1) ? *reinterpret_cast<volatile uint32_t*>(p.ar_state) + 1 : 0;
    const uint64_t ar_units = ((uint64_t)p.m * p.n) >> 2;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const uint32_t tx = p.box_m * BK * 2 + S::B_BYTES;
            // after an abort nothing new is requested, but the stages whose B tiles are already in flight still get
            // their A tiles: their barriers then complete and the loop below sees the copies land before the CTA ends
            const uint32_t todo = *s_abort ? pre : nkb;
            for (uint32_t i = 0; i < todo; ++i) {
                const uint32_t s = i % STAGES, use = i / STAGES;
                if (use > 0 && !mbar_wait(bar_empty + 8 * s, (use - 1) & 1, s_abort, p.status)) break;
                const uint32_t st = base + s * S::STAGE;
                const int k0 = (int)((kb_begin + i) * BK);
                if (i >= pre) mbar_arrive_expect_tx(bar_full + 8 * s, tx);
                tma_load_2d(st, &map_a, k0, (int)m0, bar_full + 8 * s);
                if (i >= pre) {
#pragma unroll
                    for (int h = 0; h < BN / 64; ++h)
                        tma_load_2d(st + S::A_BYTES + h * (BK * 128), &map_b, (int)(n0 + 64 * h), k0, bar_full + 8 * s);
                }
            }
            if (*s_abort)
                for (uint32_t i = 0; i < pre; ++i)
                    for (uint32_t it = 0; it < WAIT_LIMIT && !mbar_try_wait(bar_full + 8 * i, 0); ++it) __nanosleep(64);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && !*s_abort) {
            // instruction descriptor: D = f32, A = B = bf16 (format 1) or f16 (format 0), A K-major,
            // B N-major, N = BN, M = 128
            constexpr uint32_t fmt = F16 ? 0u : 1u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (uint32_t i = 0; i < nkb && ok; ++i) {
                const uint32_t s = i % STAGES, use = i / STAGES;
                ok = mbar_wait(bar_full + 8 * s, use & 1, s_abort, p.status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = base + s * S::STAGE, b_addr = a_addr + S::A_BYTES;
#pragma unroll
                for (int j = 0; j < BK / 16; ++j) {
                    // A: 16 k-elements = 32 bytes inside the swizzled 128-byte row; 8-row groups 1024 B apart
                    const uint64_t da = smem_desc(a_addr + j * 32, 16, 1024);
                    // B: 16 k-rows = two 8-row groups (1024 B apart); 64-column chunks BK*128 B apart
                    const uint64_t db = smem_desc(b_addr + j * 2048, BK * 128, 1024);
                    umma_bf16(tmem_base, da, db, idesc, (i | (uint32_t)j) != 0 ? 1u : 0u);
                }
                umma_commit(bar_empty + 8 * s);  // frees the ring slot once these MMAs have read it
            }
            if (ok) umma_commit(bar_accum);      // accumulator complete
        }
    } else {
        // ---------------- epilogue warps (TMEM lane quarter = warp % 4) ----------------
        const uint32_t quarter = warp & 3u;
        const uint32_t row = m0 + quarter * 32 + lane;
        // an earlier launch gave up on a wait: store nothing (the round trip to the status word overlaps the mainloop)
        if (warp == 2 && lane == 0 && (*reinterpret_cast<volatile uint32_t*>(p.status) & 4u)) *s_abort = 1;
        if (nkb != 0) mbar_wait(bar_accum, 0, s_abort, p.status);
        asm volatile("bar.sync 1, 128;" ::: "memory");   // all four epilogue warps see the same abort state
        const bool ok = !*s_abort;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok && p.splits == 1 && p.gated) {
            if constexpr (BN == 128) {
                const uint32_t half_n = p.n >> 1;
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    uint32_t v[32], w[32];
                    tmem_ld32(tmem_base + ((quarter * 32u) << 16) + (uint32_t)(c * 32), v);
                    tmem_ld32(tmem_base + ((quarter * 32u) << 16) + (uint32_t)(64 + c * 32), w);
                    const uint32_t col0 = (n0 >> 1) + c * 32;
                    if (row < p.m && col0 < half_n) {
                        uint16_t* dst = p.seg[0].out + (uint64_t)row * half_n + col0;
                        uint32_t packed[16];
#pragma unroll
                        for (int x = 0; x < 16; ++x) {
                            const uint16_t lo = gated_elem<F16>(__uint_as_float(v[2 * x]), __uint_as_float(w[2 * x]), p.seg[0].table);
                            const uint16_t hi = gated_elem<F16>(__uint_as_float(v[2 * x + 1]), __uint_as_float(w[2 * x + 1]), p.seg[0].table);
                            packed[x] = (uint32_t)lo | ((uint32_t)hi << 16);
                        }
#pragma unroll
                        for (int x = 0; x < 4; ++x)
                            reinterpret_cast<uint4*>(dst)[x] = make_uint4(packed[4 * x], packed[4 * x + 1], packed[4 * x + 2], packed[4 * x + 3]);
                    }
                }
            }
        } else if (ok && p.splits == 1 && (AR && p.ar_world > 1)) {
            // tensor-parallel sum in the epilogue: first push every unit of this thread's row, then
            // collect the peers' units (the NVLink latency of all pushes overlaps)
            const GemmSeg sg = p.seg[0];
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((quarter * 32u) << 16) + (uint32_t)(c * 32), v);
                    const uint32_t col0 = n0 + c * 32;
                    if (row >= p.m || col0 >= p.n) continue;
#pragma unroll 1
                    for (int x = 0; x < 8; ++x) {
                        if (col0 + 4 * x >= p.n) break;
                        const float mine4[4] = {__uint_as_float(v[4 * x]), __uint_as_float(v[4 * x + 1]), __uint_as_float(v[4 * x + 2]),
                                                __uint_as_float(v[4 * x + 3])};
                        const uint2 mine = ar_pack<F16>(mine4);
                        const uint64_t idx = (uint64_t)row * p.n + col0 + 4 * x, unit = idx >> 2;
                        if (pass == 0) {
                            ar_push(p, ar_epoch, ar_units, unit, mine);
                            continue;
                        }
                        float a4[4];
                        if (!ar_sum<F16>(p, ar_epoch, ar_units, unit, mine, a4)) {
                            atomicOr(p.status, 8u);
                            continue;
                        }
                        uint16_t h[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) h[e] = epilogue_elem<F16>(a4[e], nullptr, sg.residual, idx + e);
                        *reinterpret_cast<uint2*>(sg.out + idx) = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
                    }
                }
            }
        } else if (ok && p.splits == 1) {
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((quarter * 32u) << 16) + (uint32_t)(c * 32), v);
                const uint32_t col0 = n0 + c * 32;
                if (row < p.m && col0 < p.n) {
                    uint32_t si = 0;
                    while (si + 1 < p.nseg && col0 >= p.seg[si].col_end) ++si;
                    const GemmSeg sg = p.seg[si];
                    const uint64_t idx0 = (uint64_t)row * (sg.col_end - sg.col_begin) + (col0 - sg.col_begin);
                    uint16_t* dst = sg.out + idx0;
                    if (col0 + 32 <= sg.col_end && ((uintptr_t)dst & 15u) == 0) {
                        uint32_t w[16];
#pragma unroll
                        for (int x = 0; x < 16; ++x) {
                            uint16_t lo = epilogue_elem<F16>(__uint_as_float(v[2 * x]), sg.table, sg.residual, idx0 + 2 * x);
                            uint16_t hi = epilogue_elem<F16>(__uint_as_float(v[2 * x + 1]), sg.table, sg.residual, idx0 + 2 * x + 1);
                            w[x] = (uint32_t)lo | ((uint32_t)hi << 16);
                        }
#pragma unroll
                        for (int x = 0; x < 4; ++x)
                            reinterpret_cast<uint4*>(dst)[x] = make_uint4(w[4 * x], w[4 * x + 1], w[4 * x + 2], w[4 * x + 3]);
                    } else {
#pragma unroll
                        for (int x = 0; x < 32; ++x)
                            if (col0 + x < sg.col_end) dst[x] = epilogue_elem<F16>(__uint_as_float(v[x]), sg.table, sg.residual, idx0 + x);
                    }
                }
            }
        } else if (ok) {
            // split-K: park this CTA's f32 accumulator rows in the (now idle) ring; 16-byte units of a
            // row are XOR-swizzled with the row number so that the 32 rows of a warp do not hit one bank
            const uint32_t row_local = quarter * 32 + lane;
            if (m0 + quarter * 32 < p.m) {  // warp-uniform: the TMEM load is a whole-warp instruction
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((quarter * 32u) << 16) + (uint32_t)(c * 32), v);
                    if (row < p.m) {
#pragma unroll
                        for (int x = 0; x < 8; ++x) {
                            const uint32_t unit = (uint32_t)(c * 8 + x) ^ (row_local & 7u);
                            *reinterpret_cast<uint4*>(sm + (size_t)row_local * (BN * 4) + unit * 16) =
                                make_uint4(v[4 * x], v[4 * x + 1], v[4 * x + 2], v[4 * x + 3]);
                        }
                    }
                }
            }
        }
    }
    if (p.splits > 1) {
        // ---- cluster reduction (all threads of all CTAs of the cluster pass both barriers) ----
        __syncwarp();  // the single-lane producer / issuer loops rejoin their warps first
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp >= 2 && !*s_abort) {
            const uint32_t rank = split, S_ = p.splits, ew = warp - 2;
            const uint32_t rows_valid = min(p.m - m0, (uint32_t)BM);
            uint32_t remote[8];
#pragma unroll
            for (uint32_t sidx = 0; sidx < 8; ++sidx) {
                remote[sidx] = 0;
                if (sidx < S_) asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[sidx]) : "r"(base), "r"(sidx));
            }
            if (p.gated) {
                // BN = 128: units 0..15 of a row are gate columns, 16..31 the matching up columns
                const uint32_t half_n = p.n >> 1;
                for (uint32_t rl = rank + S_ * ew; rl < rows_valid; rl += S_ * 4) {
                    if (lane >= 16 || BN != 128) continue;
                    float4 acc[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t u = lane + 16 * h;
                        const uint32_t off = rl * (BN * 4) + ((u ^ (rl & 7u)) * 16);
                        float4 part[8];
#pragma unroll
                        for (uint32_t sidx = 0; sidx < 8; ++sidx) {
                            part[sidx] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (sidx < S_)
                                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                             : "=f"(part[sidx].x), "=f"(part[sidx].y), "=f"(part[sidx].z), "=f"(part[sidx].w)
                                             : "r"(remote[sidx] + off));
                        }
                        acc[h] = part[0];
#pragma unroll
                        for (uint32_t sidx = 1; sidx < 8; ++sidx)
                            if (sidx < S_) { acc[h].x += part[sidx].x; acc[h].y += part[sidx].y; acc[h].z += part[sidx].z; acc[h].w += part[sidx].w; }
                    }
                    const uint32_t col = (n0 >> 1) + lane * 4, grow = m0 + rl;
                    if (col < half_n) {
                        const uint16_t h0 = gated_elem<F16>(acc[0].x, acc[1].x, p.seg[0].table), h1 = gated_elem<F16>(acc[0].y, acc[1].y, p.seg[0].table);
                        const uint16_t h2 = gated_elem<F16>(acc[0].z, acc[1].z, p.seg[0].table), h3 = gated_elem<F16>(acc[0].w, acc[1].w, p.seg[0].table);
                        *reinterpret_cast<uint2*>(p.seg[0].out + (uint64_t)grow * half_n + col) =
                            make_uint2((uint32_t)h0 | ((uint32_t)h1 << 16), (uint32_t)h2 | ((uint32_t)h3 << 16));
                    }
                }
            } else if (BN == 128 && p.head_ops) {
                // One tile is one 128-wide head of one segment, and a warp holds a whole row of it (lane u: columns
                // 4u .. 4u+3). After the product is stored, the same warp rotates the stored values (rotate-half
                // RoPE: column j pairs with j +- 64, i.e. lane u with lane u ^ 16) and / or quantizes the row to i8
                // codes with one f32 scale: the arithmetic of the RotaryEmbedding and QuantizeRowsI8 calls on the
                // values the matmul stored, without their launches.
                constexpr int dt = F16 ? HOLO_DTYPE_F16 : HOLO_DTYPE_BF16;
                uint32_t si = 0;
                while (si + 1 < p.nseg && n0 >= p.seg[si].col_end) ++si;
                const GemmSeg sg = p.seg[si];
                const uint32_t width = sg.col_end - sg.col_begin, colseg = n0 - sg.col_begin + lane * 4;
                for (uint32_t rl = rank + S_ * ew; rl < rows_valid; rl += S_ * 4) {
                    const uint32_t off = rl * (BN * 4) + ((lane ^ (rl & 7u)) * 16);
                    float4 part[8];
#pragma unroll
                    for (uint32_t sidx = 0; sidx < 8; ++sidx) {
                        part[sidx] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (sidx < S_)
                            asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(part[sidx].x), "=f"(part[sidx].y), "=f"(part[sidx].z), "=f"(part[sidx].w)
                                         : "r"(remote[sidx] + off));
                    }
                    float4 acc = part[0];
#pragma unroll
                    for (uint32_t sidx = 1; sidx < 8; ++sidx)
                        if (sidx < S_) { acc.x += part[sidx].x; acc.y += part[sidx].y; acc.z += part[sidx].z; acc.w += part[sidx].w; }
                    const uint64_t grow = m0 + rl, idx = grow * width + colseg;
                    const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
                    uint16_t h[4];
#pragma unroll
                    for (int x = 0; x < 4; ++x) h[x] = epilogue_elem<F16>(a4[x], sg.table, sg.residual, idx + x);
                    *reinterpret_cast<uint2*>(sg.out + idx) = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
                    if (sg.head_op == 0) continue;
                    float v[4];
#pragma unroll
                    for (int x = 0; x < 4; ++x) v[x] = holo::widen16(h[x], dt);
                    if (sg.head_op != 3) {
                        const uint2 cw = *reinterpret_cast<const uint2*>(sg.cos + idx), sw = *reinterpret_cast<const uint2*>(sg.sin + idx);
                        const uint16_t c16[4] = {(uint16_t)(cw.x & 0xffffu), (uint16_t)(cw.x >> 16), (uint16_t)(cw.y & 0xffffu), (uint16_t)(cw.y >> 16)};
                        const uint16_t s16[4] = {(uint16_t)(sw.x & 0xffffu), (uint16_t)(sw.x >> 16), (uint16_t)(sw.y & 0xffffu), (uint16_t)(sw.y >> 16)};
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            const float other = __shfl_xor_sync(0xffffffffu, v[x], 16);
                            const float xc = __fmul_rn(v[x], holo::widen16(c16[x], dt)), os = __fmul_rn(other, holo::widen16(s16[x], dt));
                            h[x] = holo::narrow16(lane < 16 ? __fsub_rn(xc, os) : __fadd_rn(xc, os), dt);
                        }
                        *reinterpret_cast<uint2*>(sg.rope_out + idx) = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
#pragma unroll
                        for (int x = 0; x < 4; ++x) v[x] = holo::widen16(h[x], dt);   // what the store kept
                    }
                    if (sg.head_op >= 2) {
                        float amax = 0.0f;
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            const float av = v[x] < 0.0f ? -v[x] : v[x];
                            if (av > amax) amax = av;
                        }
                        for (int o = 16; o > 0; o >>= 1) {
                            const float other = __shfl_xor_sync(0xffffffffu, amax, o);
                            if (other > amax) amax = other;
                        }
                        const bool zero = amax == 0.0f;
                        const float inv = zero ? 0.0f : __fdiv_rn(127.0f, amax);
                        uint32_t packed = 0;
                        if (!zero) {
#pragma unroll
                            for (int x = 0; x < 4; ++x) {
                                const float t = __fmul_rn(v[x], inv);
                                int r = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
                                r = max(-127, min(127, r));
                                packed |= ((uint32_t)r & 0xffu) << (8 * x);
                            }
                        }
                        *reinterpret_cast<uint32_t*>(sg.codes + idx) = packed;
                        if (lane == 0) sg.scales[idx >> 7] = zero ? 0.0f : __fdiv_rn(amax, 127.0f);
                    }
                }
            } else
            for (int pass = (AR && p.ar_world > 1) ? 0 : 1; pass < 2; ++pass)
            for (uint32_t rl = rank + S_ * ew; rl < rows_valid; rl += S_ * 4) {
                for (uint32_t u = lane; u < BN / 4; u += 32) {
                    const uint32_t off = rl * (BN * 4) + ((u ^ (rl & 7u)) * 16);
                    float4 part[8];
#pragma unroll
                    for (uint32_t sidx = 0; sidx < 8; ++sidx) {
                        part[sidx] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (sidx < S_)
                            asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(part[sidx].x), "=f"(part[sidx].y), "=f"(part[sidx].z), "=f"(part[sidx].w)
                                         : "r"(remote[sidx] + off));
                    }
                    float4 acc = part[0];
#pragma unroll
                    for (uint32_t sidx = 1; sidx < 8; ++sidx)
                        if (sidx < S_) { acc.x += part[sidx].x; acc.y += part[sidx].y; acc.z += part[sidx].z; acc.w += part[sidx].w; }
                    const uint32_t col = n0 + u * 4, grow = m0 + rl;
                    if (col < p.n) {
                        uint32_t si = 0;
                        while (si + 1 < p.nseg && col >= p.seg[si].col_end) ++si;
                        const GemmSeg sg = p.seg[si];
                        const uint64_t idx = (uint64_t)grow * (sg.col_end - sg.col_begin) + (col - sg.col_begin);
                        uint16_t* dst = sg.out + idx;
                        float a4[4] = {acc.x, acc.y, acc.z, acc.w};
                        if ((AR && p.ar_world > 1)) {
                            // this rank's narrowed partial goes to the peers in the first pass; in the
                            // second the sums over the ranks replace it (single segment: idx = row * n + col)
                            const uint2 mine = ar_pack<F16>(a4);
                            if (pass == 0) {
                                ar_push(p, ar_epoch, ar_units, idx >> 2, mine);
                                continue;
                            }
                            if (!ar_sum<F16>(p, ar_epoch, ar_units, idx >> 2, mine, a4)) {
                                atomicOr(p.status, 8u);
                                continue;
                            }
                        }
                        if (col + 4 <= sg.col_end && ((uintptr_t)dst & 7u) == 0) {
                            uint16_t h[4];
#pragma unroll
                            for (int x = 0; x < 4; ++x) h[x] = epilogue_elem<F16>(a4[x], sg.table, sg.residual, idx + x);
                            *reinterpret_cast<uint2*>(dst) = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
                        } else {
#pragma unroll
                            for (int x = 0; x < 4; ++x)
                                if (col + x < sg.col_end) dst[x] = epilogue_elem<F16>(a4[x], sg.table, sg.residual, idx + x);
                        }
                    }
                }
            }
        }
        // nobody leaves (and frees its shared memory) while a neighbour may still read it
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    // everyone meets here, whatever happened above, so that TMEM is always released
    __syncwarp();  // the single-lane producer / issuer loops rejoin their warps first
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
    if ((AR && p.ar_world > 1) && threadIdx.x == 0) {
        // the launch's last CTA advances the group's epoch (every CTA has read it by then)
        const uint32_t done = atomicAdd(p.ar_state + 1, 1u);
        if (done == gridDim.x * gridDim.y * gridDim.z - 1) {
            p.ar_state[1] = 0;
            p.ar_state[0] = ar_epoch;
        }
    }
}


// ---- persistent kernel for compute-bound shapes ---------------------------------------------------
// One CTA per SM walks the 128 x 256 output tiles (tile t, t + grid, ...). A 128 x 128 tile reads 32 KiB of
// shared-memory operands per 64-deep k-block for 64 MMA clocks, which is the shared-memory bandwidth itself;
// at 128 x 256 the same A block feeds twice the columns (48 KiB for 128 clocks), so the tensor pipe is no
// longer starved by its operands. The accumulator is double-buffered in TMEM (2 x 256 columns = all 512):
// while the four epilogue warps drain tile i from one half, the issuer already accumulates tile i + 1 into
// the other, and the TMA producer runs ahead through a 4-stage ring that never drains between tiles.
//   warp 0   TMA producer (ring slot counter runs across tiles)
//   warp 1   tcgen05.mma issuer; commits ring slots back to the producer and finished accumulators to the epilogue
//   warps 2-5 epilogue: tcgen05.ld, narrow, epilogue op, store; hands the TMEM half back to the issuer
// Every wait is bounded; a wait that gives up raises the status bit, every role leaves its loop, and the
// CTA still frees its TMEM.
constexpr int PBN = 256, PSTAGES = 4;
struct PersistSmem {
    static constexpr uint32_t A_BYTES = BM * BK * 2;            // 16 KiB
    static constexpr uint32_t B_BYTES = BK * PBN * 2;           // 32 KiB
    static constexpr uint32_t STAGE = A_BYTES + B_BYTES;
    static constexpr uint32_t RING = PSTAGES * STAGE;           // 192 KiB
    static constexpr uint32_t TOTAL = RING + 256 + 1024;        // barriers, TMEM slot, abort flag; alignment slack
};

template <bool F16>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
matmul_umma_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using S = PersistSmem;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    const uint32_t bar_full = base + S::RING, bar_empty = bar_full + 8 * PSTAGES;
    const uint32_t bar_acc_full = bar_empty + 8 * PSTAGES, bar_acc_empty = bar_acc_full + 16;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(sm + S::RING + 16 * PSTAGES + 32);
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(sm + S::RING + 16 * PSTAGES + 36);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles_n = (p.n + PBN - 1) / PBN, tiles_m = (p.m + BM - 1) / BM, ntiles = tiles_n * tiles_m;

    holo_pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);   // one arrival per epilogue warp
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *s_tmem;
    holo_pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const uint32_t tx = S::A_BYTES + S::B_BYTES;
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (int)((tile / tiles_n) * BM), n0 = (int)((tile % tiles_n) * PBN);
                for (uint32_t kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const uint32_t s = it % PSTAGES, use = it / PSTAGES;
                    if (use > 0 && !mbar_wait(bar_empty + 8 * s, (use - 1) & 1, s_abort, p.status)) { ok = false; break; }
                    const uint32_t st = base + s * S::STAGE;
                    const int k0 = (int)(kb * BK);
                    mbar_arrive_expect_tx(bar_full + 8 * s, tx);
                    tma_load_2d(st, &map_a, k0, m0, bar_full + 8 * s);
#pragma unroll
                    for (int h = 0; h < PBN / 64; ++h) tma_load_2d(st + S::A_BYTES + h * (BK * 128), &map_b, n0 + 64 * h, k0, bar_full + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t fmt = F16 ? 0u : 1u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(PBN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++t) {
                const uint32_t buf = t & 1u, use = t >> 1;
                // the epilogue must have drained this half of TMEM (its previous use) before it is overwritten
                if (use > 0 && !mbar_wait(bar_acc_empty + 8 * buf, (use - 1) & 1, s_abort, p.status)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * (uint32_t)PBN;
                for (uint32_t kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const uint32_t s = it % PSTAGES;
                    if (!mbar_wait(bar_full + 8 * s, (it / PSTAGES) & 1, s_abort, p.status)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = base + s * S::STAGE, b_addr = a_addr + S::A_BYTES;
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j) {
                        const uint64_t da = smem_desc(a_addr + j * 32, 16, 1024);
                        const uint64_t db = smem_desc(b_addr + j * 2048, BK * 128, 1024);
                        umma_bf16(tmem_d, da, db, idesc, (kb | (uint32_t)j) != 0 ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * s);
                }
                if (ok) umma_commit(bar_acc_full + 8 * buf);
            }
        }
    } else {
        // ---------------- epilogue warps (TMEM lane quarter = warp % 4) ----------------
        const uint32_t quarter = warp & 3u;
        if (warp == 2 && lane == 0 && (*reinterpret_cast<volatile uint32_t*>(p.status) & 4u)) *s_abort = 1;   // an earlier launch gave up: store nothing
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t t = 0;
        for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u, use = t >> 1;
            const uint32_t m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * PBN;
            const uint32_t row = m0 + quarter * 32 + lane;
            const bool got = mbar_wait(bar_acc_full + 8 * buf, use & 1, s_abort, p.status);
            if (!got || *s_abort) break;    // the abort flag is shared: every warp of the CTA leaves its loop
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + buf * (uint32_t)PBN + ((quarter * 32u) << 16);
#pragma unroll 1
            for (int c = 0; c < PBN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_d + (uint32_t)(c * 32), v);
                const uint32_t col0 = n0 + c * 32;
                if (row < p.m && col0 < p.n) {
                    uint32_t si = 0;
                    while (si + 1 < p.nseg && col0 >= p.seg[si].col_end) ++si;
                    const GemmSeg sg = p.seg[si];
                    const uint64_t idx0 = (uint64_t)row * (sg.col_end - sg.col_begin) + (col0 - sg.col_begin);
                    uint16_t* dst = sg.out + idx0;
                    if (col0 + 32 <= sg.col_end && ((uintptr_t)dst & 15u) == 0) {
                        uint32_t w[16];
#pragma unroll
                        for (int x = 0; x < 16; ++x) {
                            const uint16_t lo = epilogue_elem<F16>(__uint_as_float(v[2 * x]), sg.table, sg.residual, idx0 + 2 * x);
                            const uint16_t hi = epilogue_elem<F16>(__uint_as_float(v[2 * x + 1]), sg.table, sg.residual, idx0 + 2 * x + 1);
                            w[x] = (uint32_t)lo | ((uint32_t)hi << 16);
                        }
#pragma unroll
                        for (int x = 0; x < 4; ++x)
                            reinterpret_cast<uint4*>(dst)[x] = make_uint4(w[4 * x], w[4 * x + 1], w[4 * x + 2], w[4 * x + 3]);
                    } else {
#pragma unroll
                        for (int x = 0; x < 32; ++x)
                            if (col0 + x < sg.col_end) dst[x] = epilogue_elem<F16>(__uint_as_float(v[x]), sg.table, sg.residual, idx0 + x);
                    }
                }
            }
            // this half of TMEM may be overwritten once all four warps have read it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_acc_empty + 8 * buf) : "memory");
        }
    }
    // everyone meets here, whatever happened above, so that TMEM is always released
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- persistent kernel on CTA pairs (tcgen05 cta_group::2) -----------------------------------------
// At 128 x 256 per CTA the product is bound by what the SMs can pull out of L2 (48 KiB of operands per
// 4.2 MFLOP). Two CTAs of a cluster share one 256 x 256 tile instead: CTA r of the pair loads rows
// [128 r, 128 r + 128) of the A block and columns [128 r, 128 r + 128) of the B block (32 KiB per CTA for the
// same 4.2 MFLOP per CTA, a third less L2 traffic), the leader CTA issues one tcgen05.mma.cta_group::2 per
// 16-deep k step which reads both CTAs' shared memory, and each CTA ends up with its own 128 rows x 256
// columns of the accumulator in its own TMEM. No multicast load is involved: every CTA fetches its own
// halves with plain tiled TMA loads, which signal the leader's barrier.
//   both CTAs  warp 0: TMA producer for its halves (waits on its own "empty" barriers, signals the leader's "full")
//   leader     warp 1: MMA issuer; tcgen05.commit multicasts "slot free" and "accumulator ready" to both CTAs
//   both CTAs  warps 2-5: epilogue from their own TMEM; hand the TMEM half back by arriving on the leader's barrier
// The accumulator is double-buffered (2 x 256 columns), the ring has 7 stages and never drains between tiles.
// Every mbarrier wait is bounded; the only unbounded waits are the two cluster barriers (after barrier set-up
// and before TMEM is released), which every thread of both CTAs reaches after bounded waits only.
constexpr int QSTAGES = 7;
struct PairSmem {
    static constexpr uint32_t A_BYTES = BM * BK * 2;            // this CTA's 128 rows: 16 KiB
    static constexpr uint32_t B_BYTES = BK * 128 * 2;           // this CTA's 128 columns: 16 KiB
    static constexpr uint32_t STAGE = A_BYTES + B_BYTES;
    static constexpr uint32_t RING = QSTAGES * STAGE;           // 224 KiB: what arrives from L2 takes 1-2 us, so every KiB in flight counts
    static constexpr uint32_t TOTAL = RING + 256 + 1024;
};
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}

// Work item w of the pair kernel: tile row, first column and width (256, or 128 for the halves of a tail tile).
struct PairItem {
    uint32_t m_tile, n0, bn;
};
__device__ __forceinline__ PairItem pair_item(const GemmParams& p, uint32_t w, uint32_t tiles_n) {
    PairItem it;
    if (w < p.tail_begin) {
        it.m_tile = w / tiles_n;
        it.n0 = (w % tiles_n) * 256;
        it.bn = 256;
    } else {
        const uint32_t h = w - p.tail_begin, tile = p.tail_begin + (h >> 1);
        it.m_tile = tile / tiles_n;
        it.n0 = (tile % tiles_n) * 256 + (h & 1u) * 128;
        it.bn = 128;
    }
    return it;
}

template <bool F16>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
matmul_umma_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using S = PairSmem;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - raw);
    const uint32_t bar_full = base + S::RING, bar_empty = bar_full + 8 * QSTAGES;
    const uint32_t bar_acc_full = bar_empty + 8 * QSTAGES, bar_acc_empty = bar_acc_full + 16;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(sm + S::RING + 16 * QSTAGES + 32);
    volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(sm + S::RING + 16 * QSTAGES + 36);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the pair is a cluster of two along grid x (the hardware pairs CTAs whose cluster rank differs in the lowest bit)
    const uint32_t rank = blockIdx.x & 1u, pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;   // rank 0 = leader
    const uint32_t tiles_n = (p.n + 255) / 256, tiles_m = (p.m + 255) / 256, ntiles = tiles_n * tiles_m;

    holo_pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < QSTAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);    // the leader's one arrive.expect_tx; the bytes come from both CTAs
            mbar_init(bar_empty + 8 * s, 1);   // one multicast commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 8);   // four epilogue warps of each CTA (used in the leader only)
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // the same warp of both CTAs allocates the pair's TMEM columns
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // the peer's loads signal the leader's barriers: nobody starts before both CTAs have set theirs up
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *s_tmem;
    holo_pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t w = pair; w < p.n_items && ok; w += npairs) {
                const PairItem item = pair_item(p, w, tiles_n);
                // this CTA's halves: rows [128 r, +128) of the A block, columns [bn/2 r, +bn/2) of the B block
                const int m0 = (int)(item.m_tile * 256 + rank * 128), n0 = (int)(item.n0 + rank * (item.bn >> 1));
                const uint32_t tx = 2u * (S::A_BYTES + (item.bn >> 1) * BK * 2);
                for (uint32_t kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const uint32_t s = it % QSTAGES, use = it / QSTAGES;
                    if (use > 0 && !mbar_wait(bar_empty + 8 * s, (use - 1) & 1, s_abort, p.status)) { ok = false; break; }
                    const uint32_t st = base + s * S::STAGE;
                    const int k0 = (int)(kb * BK);
                    if (rank == 0) mbar_arrive_expect_tx(bar_full + 8 * s, tx);
                    const uint32_t leader_bar = map_to_cta(bar_full + 8 * s, 0);
                    tma_load_2d_pair(st, &map_a, k0, m0, leader_bar);
                    tma_load_2d_pair(st + S::A_BYTES, &map_b, n0, k0, leader_bar);
                    if (item.bn == 256) tma_load_2d_pair(st + S::A_BYTES + BK * 128, &map_b, n0 + 64, k0, leader_bar);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t fmt = F16 ? 0u : 1u;
            // D = f32, A = B = bf16 / f16, A K-major, B N-major, N = 256 (128 for a tail half), M = 256 (128 rows in each CTA)
            const uint32_t idesc_base = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | ((uint32_t)(256 >> 4) << 24);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (uint32_t w = pair; w < p.n_items && ok; w += npairs, ++t) {
                const uint32_t idesc = idesc_base | ((pair_item(p, w, tiles_n).bn >> 3) << 17);
                const uint32_t buf = t & 1u, use = t >> 1;
                if (use > 0 && !mbar_wait(bar_acc_empty + 8 * buf, (use - 1) & 1, s_abort, p.status)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * 256u;
                for (uint32_t kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const uint32_t s = it % QSTAGES;
                    if (!mbar_wait(bar_full + 8 * s, (it / QSTAGES) & 1, s_abort, p.status)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = base + s * S::STAGE, b_addr = a_addr + S::A_BYTES;
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j) {
                        const uint64_t da = smem_desc(a_addr + j * 32, 16, 1024);
                        const uint64_t db = smem_desc(b_addr + j * 2048, BK * 128, 1024);
                        umma_bf16_pair(tmem_d, da, db, idesc, (kb | (uint32_t)j) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(bar_empty + 8 * s);
                }
                if (ok) umma_commit_pair(bar_acc_full + 8 * buf);
            }
        }
    } else {
        // ---------------- epilogue warps (both CTAs; TMEM lane quarter = warp % 4) ----------------
        const uint32_t quarter = warp & 3u;
        if (warp == 2 && lane == 0 && (*reinterpret_cast<volatile uint32_t*>(p.status) & 4u)) *s_abort = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t leader_acc_empty = map_to_cta(bar_acc_empty, 0);
        uint32_t t = 0;
        for (uint32_t w = pair; w < p.n_items; w += npairs, ++t) {
            const uint32_t buf = t & 1u, use = t >> 1;
            const PairItem item = pair_item(p, w, tiles_n);
            const uint32_t m0 = item.m_tile * 256 + rank * 128, n0 = item.n0;
            const uint32_t row = m0 + quarter * 32 + lane;
            const bool got = mbar_wait(bar_acc_full + 8 * buf, use & 1, s_abort, p.status);
            if (!got || *s_abort) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + buf * 256u + ((quarter * 32u) << 16);
#pragma unroll 1
            for (int c = 0; c < (int)(item.bn / 32); ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_d + (uint32_t)(c * 32), v);
                const uint32_t col0 = n0 + c * 32;
                if (row < p.m && col0 < p.n) {
                    uint32_t si = 0;
                    while (si + 1 < p.nseg && col0 >= p.seg[si].col_end) ++si;
                    const GemmSeg sg = p.seg[si];
                    const uint64_t idx0 = (uint64_t)row * (sg.col_end - sg.col_begin) + (col0 - sg.col_begin);
                    uint16_t* dst = sg.out + idx0;
                    if (col0 + 32 <= sg.col_end && ((uintptr_t)dst & 15u) == 0) {
                        uint32_t w[16];
#pragma unroll
                        for (int x = 0; x < 16; ++x) {
                            const uint16_t lo = epilogue_elem<F16>(__uint_as_float(v[2 * x]), sg.table, sg.residual, idx0 + 2 * x);
                            const uint16_t hi = epilogue_elem<F16>(__uint_as_float(v[2 * x + 1]), sg.table, sg.residual, idx0 + 2 * x + 1);
                            w[x] = (uint32_t)lo | ((uint32_t)hi << 16);
                        }
#pragma unroll
                        for (int x = 0; x < 4; ++x)
                            reinterpret_cast<uint4*>(dst)[x] = make_uint4(w[4 * x], w[4 * x + 1], w[4 * x + 2], w[4 * x + 3]);
                    } else {
#pragma unroll
                        for (int x = 0; x < 32; ++x)
                            if (col0 + x < sg.col_end) dst[x] = epilogue_elem<F16>(__uint_as_float(v[x]), sg.table, sg.residual, idx0 + x);
                    }
                }
            }
            // this half of both CTAs' TMEM may be overwritten once all eight epilogue warps of the pair have read it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(leader_acc_empty + 8 * buf) : "memory");
        }
    }
    // Nobody frees TMEM or leaves (and gives up the shared memory the pair's MMAs and barriers live in) before
    // both CTAs are through.
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Shapes the tensor-core path cannot take (row pitches that are not 16-byte multiples,
// unaligned bases), tiny problems and every f32 product: one thread per output cell running the
// reference's own per-cell recurrence, an ascending-k fused multiply-add chain (mul-then-add in
// the n % 8 column tail, cpu/simd.rs:746-799) -- bit-identical to the CPU kernel. For f32 the
// fused activation is the scalar function itself (no table exists for 32-bit patterns).
// `add_first` (MatMulAddActivation, cpu/float_kernels.rs:899-938): the residual is added before the activation and
// nothing is narrowed between the two; for 16-bit dtypes the product itself is narrowed once, as the matmul stores it.
__global__ void matmul_cell_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ out,
                                   const uint16_t* __restrict__ table, int act, const void* __restrict__ residual, uint32_t m,
                                   uint32_t k, uint32_t n, int dtype, int add_first) {
    holo_pdl_trigger();
    holo_pdl_wait();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, i = blockIdx.y;
    if (j >= n || i >= m) return;
    const bool fused = j < n - (n % 8);
    float acc = 0.0f;
    for (uint32_t kk = 0; kk < k; ++kk) {
        float av = holo::load_float(a, (uint64_t)i * k + kk, dtype), bv = holo::load_float(b, (uint64_t)kk * n + j, dtype);
        acc = fused ? __fmaf_rn(av, bv, acc) : __fadd_rn(acc, __fmul_rn(av, bv));
    }
    const uint64_t idx = (uint64_t)i * n + j;
    if (add_first) {
        if (dtype == HOLO_DTYPE_F32) {
            acc = __fadd_rn(acc, reinterpret_cast<const float*>(residual)[idx]);
            reinterpret_cast<float*>(out)[idx] = holo::lut_act_ref(act, acc);
        } else {
            const float v = __fadd_rn(holo::widen16(holo::narrow16(acc, dtype), dtype), holo::widen16(reinterpret_cast<const uint16_t*>(residual)[idx], dtype));
            reinterpret_cast<uint16_t*>(out)[idx] = holo::narrow16(holo::lut_act_ref(act, v), dtype);
        }
        return;
    }
    if (dtype == HOLO_DTYPE_F32) {
        if (act >= 0) acc = holo::lut_act_ref(act, acc);
        if (residual) acc = __fadd_rn(acc, reinterpret_cast<const float*>(residual)[idx]);
        reinterpret_cast<float*>(out)[idx] = acc;
    } else {
        const uint16_t* res16 = reinterpret_cast<const uint16_t*>(residual);
        reinterpret_cast<uint16_t*>(out)[idx] = dtype == HOLO_DTYPE_F16 ? epilogue_elem<true>(acc, table, res16, idx) : epilogue_elem<false>(acc, table, res16, idx);
    }
}

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

int32_t make_map_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t es[2] = {1, 1};
    CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: cuTensorMapEncodeTiled (matmul) returned %d", (int)r);
    return HOLO_OK;
}

template <int BN, int STAGES, int A_ROWS, bool F16, bool AR>
int32_t launch_umma_ar(holo_b200_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid) {
    using S = GemmSmem<BN, STAGES, A_ROWS>;
    static thread_local int configured_device = -1;
    if (configured_device != ctx->device) {
        HOLO_CUDA(cudaFuncSetAttribute(matmul_bf16_umma_kernel<BN, STAGES, A_ROWS, F16, AR>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
        configured_device = ctx->device;
    }
    // the K slices of one output tile form a cluster along grid z
    HOLO_CUDA(holo_launch_kernel(ctx, matmul_bf16_umma_kernel<BN, STAGES, A_ROWS, F16, AR>, grid, dim3(GEMM_THREADS), S::TOTAL, p.splits, ma, mb, p));
    ctx->launches++;
    return HOLO_OK;
}

template <int BN, int STAGES, int A_ROWS, bool F16>
int32_t launch_umma_dt(holo_b200_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid) {
    if (p.ar_world > 1) return launch_umma_ar<BN, STAGES, A_ROWS, F16, true>(ctx, ma, mb, p, grid);
    return launch_umma_ar<BN, STAGES, A_ROWS, F16, false>(ctx, ma, mb, p, grid);
}

template <int BN, int STAGES, int A_ROWS>
int32_t launch_umma(holo_b200_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid) {
    if (p.dtype == HOLO_DTYPE_F16) return launch_umma_dt<BN, STAGES, A_ROWS, true>(ctx, ma, mb, p, grid);
    return launch_umma_dt<BN, STAGES, A_ROWS, false>(ctx, ma, mb, p, grid);
}

}  // namespace

static int lut_id_of_fused(uint8_t fused_act) {
    return fused_act == HOLO_FUSED_GELU ? HOLO_LUT_GELU : fused_act == HOLO_FUSED_SILU ? HOLO_LUT_SILU
         : fused_act == HOLO_FUSED_SIGMOID ? HOLO_LUT_SIGMOID : fused_act == HOLO_FUSED_TANH ? HOLO_LUT_TANH : HOLO_LUT_EXP;
}

static int32_t act_table(holo_b200_ctx* ctx, uint8_t fused_act, uint8_t dtype, const uint16_t** table) {
    *table = nullptr;
    if (fused_act) {
        int act = fused_act == HOLO_FUSED_GELU ? HOLO_LUT_GELU : fused_act == HOLO_FUSED_SILU ? HOLO_LUT_SILU
                : fused_act == HOLO_FUSED_SIGMOID ? HOLO_LUT_SIGMOID : fused_act == HOLO_FUSED_TANH ? HOLO_LUT_TANH : HOLO_LUT_EXP;
        HOLO_TRY(holo_lut_table(ctx, (uint8_t)act, dtype, table));
    }
    return HOLO_OK;
}

int32_t holo_launch_matmul(holo_b200_ctx* ctx, const void* a, const void* b, void* out, uint32_t m, uint32_t k, uint32_t n,
                           uint8_t dtype, uint8_t fused_act, const void* residual, bool b_constant) {
    HoloMatmulSeg sg = {out, residual, n, fused_act};
    sg.b_constant = b_constant ? 1 : 0;
    return holo_launch_matmul_multi(ctx, a, b, m, k, n, dtype, &sg, 1);
}

int32_t holo_launch_matmul_add_activation(holo_b200_ctx* ctx, const void* a, const void* b, void* out, uint32_t m, uint32_t k, uint32_t n,
                                          uint8_t dtype, uint8_t fused_act, const void* residual) {
    if (m > 65535) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul m %u on the per-cell path", m);
    HOLO_CUDA(holo_launch_kernel(ctx, matmul_cell_kernel, dim3((n + 127) / 128, m), dim3(128), 0, 1, a, b, out, (const uint16_t*)nullptr,
                                 lut_id_of_fused(fused_act), residual, m, k, n, (int)dtype, 1));
    ctx->launches++;
    return HOLO_OK;
}

// C[:, segment i] = epilogue_i(A . B[:, segment i]) for 1..3 column segments of one [k, n] B.
// Whether the segments' head_op requests can ride this product: the tensor-core path with one row tile, K
// split at least two ways inside a cluster, every segment a whole number of 128-column heads, no gate, no
// tensor-parallel sum. The session asks before it folds a RotaryEmbedding / QuantizeRowsI8 into a product.
bool holo_matmul_head_ops_ok(uint32_t m, uint32_t k, uint32_t n, uint8_t dtype, const HoloMatmulSeg* segs, uint32_t nseg) {
    if (dtype != HOLO_DTYPE_BF16 && dtype != HOLO_DTYPE_F16) return false;
    if (m == 0 || m > (uint32_t)BM || k < 2 * BK || (k % 8) != 0 || (n % 128) != 0 || nseg < 1 || nseg > MAX_SEGS) return false;
    if ((uint64_t)m * n * k < (1ull << 18) || encode_tiled_fn() == nullptr) return false;
    // the compute-bound kernels have no head epilogue (they need two row tiles, excluded above)
    for (uint32_t i = 0; i < nseg; ++i) {
        if ((segs[i].width % 128) != 0 || segs[i].gated || segs[i].all_reduce) return false;
        if (segs[i].head_op > 3) return false;
        if (segs[i].head_op == 1 || segs[i].head_op == 2)
            if (!segs[i].cos || !segs[i].sin || !segs[i].rope_out || (((uintptr_t)segs[i].cos | (uintptr_t)segs[i].sin | (uintptr_t)segs[i].rope_out) & 7u)) return false;
        if (segs[i].head_op >= 2)
            if (!segs[i].codes || !segs[i].scales || ((uintptr_t)segs[i].codes & 3u) || ((uintptr_t)segs[i].scales & 3u)) return false;
        if (segs[i].head_op && ((uintptr_t)segs[i].out & 7u)) return false;
    }
    return true;
}

int32_t holo_launch_matmul_multi(holo_b200_ctx* ctx, const void* a, const void* b, uint32_t m, uint32_t k, uint32_t n,
                                 uint8_t dtype, const HoloMatmulSeg* segs, uint32_t nseg) {
    if (nseg < 1 || nseg > MAX_SEGS) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul segment count %u", nseg);
    GemmSeg gs[MAX_SEGS] = {};
    uint32_t col = 0;
    bool head_ops = false;
    for (uint32_t i = 0; i < nseg; ++i) {
        if (dtype != HOLO_DTYPE_F32) HOLO_TRY(act_table(ctx, segs[i].fused_act, dtype, &gs[i].table));
        gs[i].out = (uint16_t*)segs[i].out;
        gs[i].residual = (const uint16_t*)segs[i].residual;
        gs[i].col_begin = col;
        col += segs[i].width;
        gs[i].col_end = col;
        if (i + 1 < nseg && (col % 32) != 0) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul segment boundary %u is not a multiple of 32", col);
        gs[i].head_op = segs[i].head_op;
        gs[i].cos = (const uint16_t*)segs[i].cos;
        gs[i].sin = (const uint16_t*)segs[i].sin;
        gs[i].rope_out = (uint16_t*)segs[i].rope_out;
        gs[i].codes = segs[i].codes;
        gs[i].scales = segs[i].scales;
        head_ops |= segs[i].head_op != 0;
    }
    if (head_ops && !holo_matmul_head_ops_ok(m, k, n, dtype, segs, nseg))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul head epilogue needs m <= 128, k >= 128 and 128-column segments");
    const bool gated = segs[0].gated != 0;
    if (gated) {
        if (nseg != 1 || (segs[0].width % 64) != 0 || dtype == HOLO_DTYPE_F32)
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: gated matmul takes one 16-bit segment whose width is a multiple of 64");
        col *= 2;
        gs[0].col_end = col;
    }
    if (col != n) return holo_fail(HOLO_ERR_SHAPE_MISMATCH, "shape mismatch: matmul segments cover %u of %u columns", col, n);
    const uint16_t* table = gs[0].table;
    const void* residual = gs[0].residual;
    void* out = gs[0].out;
    const bool tma_ok = dtype != HOLO_DTYPE_F32 && (k % 8) == 0 && (n % 8) == 0 && (((uintptr_t)a | (uintptr_t)b) & 15u) == 0 && encode_tiled_fn() != nullptr;
    const bool tiny = (uint64_t)m * n * k < (1ull << 18);
    if ((nseg > 1 || gated) && (!tma_ok || tiny))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: merged matmul needs the tensor-core path");
    const bool cell_path = !tma_ok || tiny || getenv("HOLO_GEMM_FORCE_CELL");
    if (cell_path && segs[0].all_reduce && ctx->tp_world > 1) {
        // the per-cell kernel has no exchange of its own: product first, then the all-reduce launch
        HoloMatmulSeg plain = segs[0];
        plain.all_reduce = 0;
        plain.residual = nullptr;
        HOLO_TRY(holo_launch_matmul_multi(ctx, a, b, m, k, n, dtype, &plain, 1));
        return holo_all_reduce_add(ctx, segs[0].out, segs[0].residual, segs[0].out, (uint64_t)m * n, dtype);
    }
    if (cell_path) {
        dim3 grid((n + 127) / 128, m);
        if (m > 65535) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul m %u on the per-cell path", m);
        HOLO_CUDA(holo_launch_kernel(ctx, matmul_cell_kernel, dim3(grid), dim3(128), 0, 1, a, b, out, table,
                                     segs[0].fused_act ? lut_id_of_fused(segs[0].fused_act) : -1, residual, m, k, n, (int)dtype, 0));
        HOLO_CUDA(cudaGetLastError());
        ctx->launches++;
        return HOLO_OK;
    }
    const uint32_t kblocks = (k + BK - 1) / BK, mtiles = (m + BM - 1) / BM;
    const uint32_t slots = 2u * (uint32_t)ctx->sm_count;
    // Compute-bound shapes (at least one 128 x 256 tile per SM): the persistent kernel.
    {
        const uint32_t ptiles = mtiles * ((n + PBN - 1) / PBN);
        bool persistent = mtiles >= 2 && ptiles >= (uint32_t)ctx->sm_count && !gated && !(segs[0].all_reduce && ctx->tp_world > 1);
        if (const char* e = getenv("HOLO_GEMM_PERSISTENT")) persistent = persistent && atoi(e) != 0;
        // 256 x 256 tiles on CTA pairs when there is at least one per pair of SMs
        const uint32_t qtiles = ((m + 255) / 256) * ((n + 255) / 256), pairs = (uint32_t)ctx->sm_count / 2;
        bool paired = persistent && qtiles >= pairs;
        if (const char* e = getenv("HOLO_GEMM_PAIR")) paired = paired && atoi(e) != 0;
        if (paired) {
            GemmParams p;
            memset(&p, 0, sizeof p);
            for (uint32_t i = 0; i < MAX_SEGS; ++i) p.seg[i] = gs[i];
            p.nseg = nseg;
            p.status = ctx->dev_status;
            p.m = m; p.n = n; p.k = k; p.kblocks = kblocks; p.splits = 1;
            p.box_m = BM;
            p.dtype = dtype;
            CUtensorMap ma, mb;
            HOLO_TRY(make_map_2d(&ma, a, k, m, BK, BM));
            HOLO_TRY(make_map_2d(&mb, b, n, k, 64, BK));
            static thread_local int configured_pair[2] = {-1, -1};
            static thread_local int resident_pairs[2] = {0, 0};
            const int which = dtype == HOLO_DTYPE_F16 ? 1 : 0;
            if (configured_pair[which] != ctx->device) {
                if (which) HOLO_CUDA(cudaFuncSetAttribute(matmul_umma_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL));
                else HOLO_CUDA(cudaFuncSetAttribute(matmul_umma_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL));
                // how many pairs the chip can hold at once (a GPC with an odd number of SMs leaves one unpaired)
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(2 * pairs, 1, 1);
                cfg.blockDim = dim3(GEMM_THREADS);
                cfg.dynamicSmemBytes = PairSmem::TOTAL;
                cudaLaunchAttribute at;
                at.id = cudaLaunchAttributeClusterDimension;
                at.val.clusterDim.x = 2;
                at.val.clusterDim.y = 1;
                at.val.clusterDim.z = 1;
                cfg.attrs = &at;
                cfg.numAttrs = 1;
                int nclusters = 0;
                cudaError_t oe = which ? cudaOccupancyMaxActiveClusters(&nclusters, matmul_umma_pair_kernel<true>, &cfg)
                                       : cudaOccupancyMaxActiveClusters(&nclusters, matmul_umma_pair_kernel<false>, &cfg);
                if (oe != cudaSuccess || nclusters <= 0) {
                    cudaGetLastError();
                    nclusters = (int)pairs;
                }
                resident_pairs[which] = nclusters;
                configured_pair[which] = ctx->device;
            }
            uint32_t grid = qtiles < pairs ? qtiles : pairs;
            if (grid > (uint32_t)resident_pairs[which]) grid = (uint32_t)resident_pairs[which];
            if (const char* e = getenv("HOLO_GEMM_PAIR_GRID")) grid = (uint32_t)atoi(e) > 0 ? (uint32_t)atoi(e) : grid;
            // The last, partial round: when its tiles cut in two still fit one round, run them as 256 x 128 halves
            // (every pair busy for half a tile's time instead of some pairs for a whole one). Same k order per cell.
            const uint32_t rest = qtiles % grid;
            const bool split_tail = rest != 0 && 2 * rest <= grid && !getenv("HOLO_GEMM_NO_TAIL_SPLIT");
            p.tail_begin = split_tail ? qtiles - rest : qtiles;
            p.n_items = split_tail ? qtiles + rest : qtiles;
            // the two CTAs of a pair are a cluster along grid x
            if (which) HOLO_CUDA(holo_launch_kernel_cluster(ctx, matmul_umma_pair_kernel<true>, dim3(2 * grid), dim3(GEMM_THREADS), PairSmem::TOTAL, 2u, 1u, ma, mb, p));
            else HOLO_CUDA(holo_launch_kernel_cluster(ctx, matmul_umma_pair_kernel<false>, dim3(2 * grid), dim3(GEMM_THREADS), PairSmem::TOTAL, 2u, 1u, ma, mb, p));
            ctx->launches++;
            return HOLO_OK;
        }
        if (persistent) {
            GemmParams p;
            memset(&p, 0, sizeof p);
            for (uint32_t i = 0; i < MAX_SEGS; ++i) p.seg[i] = gs[i];
            p.nseg = nseg;
            p.status = ctx->dev_status;
            p.m = m; p.n = n; p.k = k; p.kblocks = kblocks; p.splits = 1;
            p.box_m = BM;
            p.dtype = dtype;
            CUtensorMap ma, mb;
            HOLO_TRY(make_map_2d(&ma, a, k, m, BK, BM));
            HOLO_TRY(make_map_2d(&mb, b, n, k, 64, BK));
            const uint32_t grid = ptiles < (uint32_t)ctx->sm_count ? ptiles : (uint32_t)ctx->sm_count;
            static thread_local int configured_device[2] = {-1, -1};
            const int which = dtype == HOLO_DTYPE_F16 ? 1 : 0;
            if (configured_device[which] != ctx->device) {
                if (which) HOLO_CUDA(cudaFuncSetAttribute(matmul_umma_persistent_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PersistSmem::TOTAL));
                else HOLO_CUDA(cudaFuncSetAttribute(matmul_umma_persistent_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PersistSmem::TOTAL));
                configured_device[which] = ctx->device;
            }
            if (which) HOLO_CUDA(holo_launch_kernel(ctx, matmul_umma_persistent_kernel<true>, dim3(grid), dim3(GEMM_THREADS), PersistSmem::TOTAL, 1, ma, mb, p));
            else HOLO_CUDA(holo_launch_kernel(ctx, matmul_umma_persistent_kernel<false>, dim3(grid), dim3(GEMM_THREADS), PersistSmem::TOTAL, 1, ma, mb, p));
            ctx->launches++;
            return HOLO_OK;
        }
    }
    // Tile width and K split. Compute-bound shapes (many tiles) take 128-wide tiles and no
    // split. HBM-bound skinny shapes want 128..slots co-resident CTAs sharing the memory
    // system: narrow tiles first, then a K split whose f32 partials stay small.
    // Tile width and K split. Compute-bound shapes (many row tiles) take 128-wide tiles, no split.
    // One-row-tile shapes (decode) are HBM-bound: loaded HBM latency is 2-3 us, so 15-20 MB of
    // weight bytes must be in flight across the chip. Measured on B200: with >= ~200 128-wide
    // tiles, or >= one 64-wide tile per SM, no split is best (every CTA walks K in step with its
    // neighbours, which keeps DRAM pages open); narrower outputs split K up to 8 ways inside a
    // thread-block cluster, which reduces the slices through distributed shared memory.
    int bn = 128;
    uint32_t splits = 1;
    const uint32_t tiles128 = mtiles * ((n + 127) / 128), tiles64 = mtiles * ((n + 63) / 64);
    if (mtiles == 1 && tiles128 < 200) {
        // 128-wide tiles read 256-byte weight rows instead of 128-byte ones; when two K slices of them still fit one
        // wave, that beats a 64-wide tile per SM (16 x 4096 x 14336: 26.0 -> 23.3 us)
        const uint32_t fit128 = tiles128 ? slots / tiles128 : 0;
        if (tiles64 >= (uint32_t)ctx->sm_count && fit128 >= 2 && kblocks >= 8 && !getenv("HOLO_GEMM_OLD_NARROW")) {
            bn = 128;
            splits = 2;   // three slices (288 CTAs in clusters of 3) did not all become resident: 64 x 4096 x 12288 took 32.6 us against 25.3
        } else if (tiles64 >= (uint32_t)ctx->sm_count) {
            bn = 64;
        } else {
            bn = tiles128 >= 16 ? 128 : 64;
            const uint32_t tiles = bn == 128 ? tiles128 : tiles64;
            uint32_t target = 240;   // CTAs aimed at; measured on the decoder step: 240 beats 192, 224 and 256 (1.735 / 1.745 / 1.741 / 1.779 ms)
            if (const char* e = getenv("HOLO_GEMM_CTA_TARGET")) target = (uint32_t)atoi(e) > 0 ? (uint32_t)atoi(e) : target;
            splits = (target + tiles - 1) / tiles;
            if (splits > 8) splits = 8;
            // k-blocks a slice keeps at least. Two: the 1/4 and 1/8 shards of the decoder's row-parallel products (K = 1024,
            // 512) then still spread over 64-128 CTAs; with eight they ran on 32 (measured on one GPU over a rank's shard of
            // the decoder step: 0.724 -> 0.648 ms at 1/8, 0.901 -> 0.822 ms at 1/4; one k-block per slice was no better)
            uint32_t min_kb = 2;
            if (const char* e = getenv("HOLO_GEMM_MIN_KB")) min_kb = (uint32_t)atoi(e) > 0 ? (uint32_t)atoi(e) : min_kb;
            if (splits > kblocks / min_kb) splits = kblocks / min_kb ? kblocks / min_kb : 1;
        }
    } else if (tiles128 < slots / 2) {
        bn = tiles64 <= slots ? 64 : 128;
    }
    if (const char* e = getenv("HOLO_GEMM_BN")) bn = atoi(e) == 64 ? 64 : atoi(e) == 256 ? 256 : 128;
    if (gated && bn != 128) {   // the gate / up pairing is per 128-wide tile
        bn = 128;
        splits = tiles128 >= 148 ? 1 : (192 + tiles128 - 1) / tiles128;
        if (splits > 8) splits = 8;
        if (splits > kblocks / 8) splits = kblocks / 8 ? kblocks / 8 : 1;
    }
    if (const char* e = getenv("HOLO_GEMM_SPLITS")) splits = (uint32_t)atoi(e) > 0 ? (uint32_t)atoi(e) : 1;
    if (head_ops) {
        // the per-head epilogue lives in the cluster reduction of 128-wide tiles (one head per tile)
        if (bn != 128) {
            bn = 128;
            splits = (240 + tiles128 - 1) / tiles128;
            if (splits > kblocks / 8) splits = kblocks / 8 ? kblocks / 8 : 1;
        }
        if (splits < 2) splits = 2;
    }
    if (splits > kblocks) splits = kblocks;
    if (splits > 8) splits = 8;  // one cluster (portable size) per output tile
    if (mtiles > 65535 || splits > 65535) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul grid too large");

    // Tensor-parallel sum in the epilogue: needs the peer-memory transport, a single plain 16-bit
    // segment, a message that fits the one-shot mailbox regions, and every CTA of the launch resident
    // at once (a CTA waits for the same tile's CTAs on the other GPUs; with more CTAs than fit, a
    // waiting first wave here could face a second wave there). Otherwise the matmul stores its
    // narrowed partial and the all-reduce kernel follows.
    const bool want_ar = segs[0].all_reduce != 0 && ctx->tp_world > 1;
    // Opt-in (HOLO_TP_FUSED_GEMM; two ranks, or any group size with HOLO_TP_FUSED_GEMM_ANY_WORLD): measured on two
    // GPUs the product followed by the all-reduce kernel is faster (1.376 against 1.456 ms per decoder step), because
    // the fused launch must trim its K split to keep every CTA resident and its tiles wait on the peer's tiles.
    bool fused_ar = want_ar && ctx->tp_p2p && nseg == 1 && !gated && !segs[0].fused_act && (n % 4) == 0 &&
                    4ull * (uint64_t)ctx->tp_world * m * n <= P2P_ONESHOT_BYTES &&
                    ((ctx->tp_world == 2 && getenv("HOLO_TP_FUSED_GEMM")) || getenv("HOLO_TP_FUSED_GEMM_ANY_WORLD"));
    if (fused_ar) {
        // one CTA per SM is always resident, clusters included: trim the K split to stay within that
        const uint32_t tiles = ((n + bn - 1) / bn) * mtiles;
        if (tiles > (uint32_t)ctx->sm_count) fused_ar = false;
        else if (tiles * splits > (uint32_t)ctx->sm_count) splits = (uint32_t)ctx->sm_count / tiles;
    }
    if (want_ar && !fused_ar) {
        HoloMatmulSeg plain = segs[0];
        plain.all_reduce = 0;
        plain.residual = nullptr;
        HOLO_TRY(holo_launch_matmul_multi(ctx, a, b, m, k, n, dtype, &plain, 1));
        return holo_all_reduce_add(ctx, segs[0].out, segs[0].residual, segs[0].out, (uint64_t)m * n, dtype);
    }
    GemmParams p;
    p.ar_world = 0;
    p.ar_rank = 0;
    p.ar_state = nullptr;
    for (int r = 0; r < 8; ++r) p.ar_mailbox[r] = nullptr;
    if (fused_ar) {
        p.ar_world = (uint32_t)ctx->tp_world;
        p.ar_rank = (uint32_t)ctx->tp_rank;
        p.ar_state = ctx->tp_epochs;
        for (int r = 0; r < 8; ++r) p.ar_mailbox[r] = ctx->tp_mailbox[r];
    }
    for (uint32_t i = 0; i < MAX_SEGS; ++i) p.seg[i] = gs[i];
    p.nseg = nseg;
    p.status = ctx->dev_status;
    p.m = m; p.n = n; p.k = k; p.kblocks = kblocks; p.splits = splits;
    p.box_m = m < (uint32_t)BM ? m : (uint32_t)BM;
    p.dtype = dtype;
    p.gated = gated ? 1u : 0u;
    p.head_ops = head_ops ? 1u : 0u;
    p.b_constant = segs[0].b_constant && !getenv("HOLO_GEMM_NO_EARLY_B") ? 1u : 0u;
    CUtensorMap ma, mb;
    HOLO_TRY(make_map_2d(&ma, a, k, m, BK, p.box_m));
    HOLO_TRY(make_map_2d(&mb, b, n, k, 64, BK));
    dim3 grid((n + bn - 1) / bn, mtiles, splits);
    if (bn == 256) {
        if (m <= 16) HOLO_TRY((launch_umma<256, 6, 16>(ctx, ma, mb, p, grid)));
        else if (m <= 64) HOLO_TRY((launch_umma<256, 5, 64>(ctx, ma, mb, p, grid)));
        else HOLO_TRY((launch_umma<256, 4, 128>(ctx, ma, mb, p, grid)));
    } else if (bn == 128) {
        if (m <= 16) HOLO_TRY((launch_umma<128, 5, 16>(ctx, ma, mb, p, grid)));
        else if (m <= 64) HOLO_TRY((launch_umma<128, 4, 64>(ctx, ma, mb, p, grid)));
        else HOLO_TRY((launch_umma<128, 3, 128>(ctx, ma, mb, p, grid)));
    } else {
        if (m <= 16) HOLO_TRY((launch_umma<64, 9, 16>(ctx, ma, mb, p, grid)));
        else if (m <= 64) HOLO_TRY((launch_umma<64, 6, 64>(ctx, ma, mb, p, grid)));
        else HOLO_TRY((launch_umma<64, 4, 128>(ctx, ma, mb, p, grid)));
    }
    return HOLO_OK;
}
