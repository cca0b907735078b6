// 16-bit LUT activation dispatch: out[i] = table[in[i]] over 65536-entry u16 tables.
// Replaces crates/hologram-compute/src/cpu/lut.rs (build_table :43-67, unary_lut :76-98).
//
// The stream kernel is HBM-bound: 2 B read + 2 B written per element. One persistent CTA per
// SM stages the 128 KiB table into shared memory once, then walks the input with 128-bit
// coalesced loads, does eight shared-memory lookups per vector and writes 128-bit stores.
#include "common.h"
#include "numerics.cuh"

namespace {

// table[bits] = narrow(f(widen(bits))), one thread per bit pattern (cpu/lut.rs:43-67).
__global__ void build_table_kernel(uint16_t* table, int act, int dtype) {
    uint32_t bits = blockIdx.x * blockDim.x + threadIdx.x;
    if (bits >= 65536u) return;
    float x = holo::widen16((uint16_t)bits, dtype);
    float y = holo::lut_act_ref(act, x);
    table[bits] = holo::narrow16(y, dtype);
}

constexpr int LUT_THREADS = 1024;
constexpr int LUT_UNROLL = 4;
constexpr int TABLE_BYTES = 65536 * 2;

__device__ __forceinline__ uint32_t lookup2(const uint16_t* tab, uint32_t w) {
    uint32_t lo = tab[w & 0xffffu];
    uint32_t hi = tab[w >> 16];
    return lo | (hi << 16);
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Persistent stream kernel. `in`/`out` are 16-byte aligned; nvec = n / 8 full vectors; the
// n % 8 tail elements are handled by the first CTA.
__global__ void __launch_bounds__(LUT_THREADS, 1)
lut_stream_kernel(const uint16_t* __restrict__ table, const uint16_t* __restrict__ in, uint16_t* __restrict__ out,
                  uint64_t n) {
    extern __shared__ __align__(16) uint16_t s_tab[];
    const uint4* in4 = reinterpret_cast<const uint4*>(in);
    uint4* out4 = reinterpret_cast<uint4*>(out);
    const uint64_t nvec = n >> 3;
    const uint64_t chunk = (uint64_t)LUT_THREADS * LUT_UNROLL;
    uint64_t base = (uint64_t)blockIdx.x * chunk;
    const uint64_t stride = (uint64_t)gridDim.x * chunk;

    // Issue the first batch of input loads before staging the table so their latency
    // overlaps the table copy.
    uint4 v[LUT_UNROLL];
#pragma unroll
    for (int u = 0; u < LUT_UNROLL; ++u) {
        uint64_t i = base + (uint64_t)u * LUT_THREADS + threadIdx.x;
        if (i < nvec) v[u] = ld_stream(in4 + i);
    }
    {
        const uint4* t4 = reinterpret_cast<const uint4*>(table);
        uint4* s4 = reinterpret_cast<uint4*>(s_tab);
#pragma unroll
        for (int i = 0; i < TABLE_BYTES / 16 / LUT_THREADS; ++i)
            s4[i * LUT_THREADS + threadIdx.x] = __ldg(t4 + i * LUT_THREADS + threadIdx.x);
    }
    __syncthreads();

    while (base < nvec) {
        const uint64_t next = base + stride;
        uint4 nv[LUT_UNROLL];
#pragma unroll
        for (int u = 0; u < LUT_UNROLL; ++u) {
            uint64_t i = next + (uint64_t)u * LUT_THREADS + threadIdx.x;
            if (i < nvec) nv[u] = ld_stream(in4 + i);
        }
#pragma unroll
        for (int u = 0; u < LUT_UNROLL; ++u) {
            uint64_t i = base + (uint64_t)u * LUT_THREADS + threadIdx.x;
            if (i < nvec) {
                uint4 r;
                r.x = lookup2(s_tab, v[u].x);
                r.y = lookup2(s_tab, v[u].y);
                r.z = lookup2(s_tab, v[u].z);
                r.w = lookup2(s_tab, v[u].w);
                st_stream(out4 + i, r);
            }
        }
#pragma unroll
        for (int u = 0; u < LUT_UNROLL; ++u) v[u] = nv[u];
        base = next;
    }
    if (blockIdx.x == 0) {
        uint64_t i = (nvec << 3) + threadIdx.x;
        if (i < n) out[i] = s_tab[in[i]];
    }
}

// Small or unaligned inputs: gather straight from the global table (L1/L2 resident).
__global__ void lut_gather_kernel(const uint16_t* __restrict__ table, const uint16_t* __restrict__ in,
                                  uint16_t* __restrict__ out, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __ldg(table + in[i]);
}

// Aligned, medium-size inputs: one 128-bit vector per thread, table read through L1.
__global__ void lut_gather_vec_kernel(const uint16_t* __restrict__ table, const uint16_t* __restrict__ in,
                                      uint16_t* __restrict__ out, uint64_t n) {
    const uint64_t nvec = n >> 3;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < nvec) {
        uint4 v = reinterpret_cast<const uint4*>(in)[i];
        uint4 r;
        r.x = __ldg(table + (v.x & 0xffffu)) | ((uint32_t)__ldg(table + (v.x >> 16)) << 16);
        r.y = __ldg(table + (v.y & 0xffffu)) | ((uint32_t)__ldg(table + (v.y >> 16)) << 16);
        r.z = __ldg(table + (v.z & 0xffffu)) | ((uint32_t)__ldg(table + (v.z >> 16)) << 16);
        r.w = __ldg(table + (v.w & 0xffffu)) | ((uint32_t)__ldg(table + (v.w >> 16)) << 16);
        reinterpret_cast<uint4*>(out)[i] = r;
    }
    if (i == 0) {
        for (uint64_t t = nvec << 3; t < n; ++t) out[t] = __ldg(table + in[t]);
    }
}

}  // namespace

// Lazily build (on the device) and cache the table for (act, dtype), as the reference's
// OnceLock cache does on the host (cpu/lut.rs:38-72).
int32_t holo_lut_table(holo_b200_ctx* ctx, uint8_t act, uint8_t dtype, const uint16_t** table) {
    if (act >= HOLO_LUT_COUNT) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "lut: unknown activation id %u", act);
    if (dtype != HOLO_DTYPE_F16 && dtype != HOLO_DTYPE_BF16)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "lut: dtype %u is not a 16-bit float", dtype);
    int di = dtype == HOLO_DTYPE_F16 ? 0 : 1;
    if (!ctx->lut[act][di]) {
        uint16_t* t = nullptr;
        HOLO_CUDA(cudaMalloc(&t, TABLE_BYTES));
        build_table_kernel<<<65536 / 256, 256, 0, ctx->stream>>>(t, act, dtype);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            cudaFree(t);
            return holo_cuda_fail(e, "build_table_kernel");
        }
        ctx->launches++;
        ctx->lut[act][di] = t;
    }
    *table = ctx->lut[act][di];
    return HOLO_OK;
}

int32_t holo_launch_lut(holo_b200_ctx* ctx, const uint16_t* table, const uint16_t* in, uint16_t* out, uint64_t n) {
    if (n == 0) return HOLO_OK;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const uint64_t nvec = n >> 3;
    if (aligned && n >= (1ull << 21)) {
        static thread_local int configured_device = -1;
        if (configured_device != ctx->device) {
            HOLO_CUDA(cudaFuncSetAttribute(lut_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TABLE_BYTES));
            configured_device = ctx->device;
        }
        const uint64_t chunk = (uint64_t)LUT_THREADS * LUT_UNROLL;
        uint64_t want = (nvec + chunk - 1) / chunk;
        int grid = (int)(want < (uint64_t)ctx->sm_count ? want : (uint64_t)ctx->sm_count);
        lut_stream_kernel<<<grid, LUT_THREADS, TABLE_BYTES, ctx->stream>>>(table, in, out, n);
    } else if (aligned && nvec > 0) {
        uint64_t blocks = (nvec + 255) / 256;
        lut_gather_vec_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(table, in, out, n);
    } else {
        uint64_t blocks = (n + 255) / 256;
        if (blocks > 65535ull * 16) blocks = 65535ull * 16;
        lut_gather_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(table, in, out, n);
    }
    HOLO_CUDA(cudaGetLastError());
    ctx->launches++;
    return HOLO_OK;
}
