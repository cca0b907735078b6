// C ABI entry points: context, device workspace, and the `Backend::dispatch` replacement.
// Validation mirrors the reference CPU kernels: geometry and slot extents are checked before
// anything is enqueued, failures are loud (negative status + thread-local message), nothing
// is silently truncated or zero-filled (crates/hologram-compute/src/error.rs, cpu/lut.rs:84-92).
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <stdlib.h>

#include "common.h"

// ---- thread-local error state (hologram-ffi src/lib.rs:48-92 convention) --------------------
static thread_local char g_err[512] = "";
static thread_local uint32_t g_err_slot = HOLO_NO_SLOT;

int32_t holo_fail(int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}
int32_t holo_fail_slot(uint32_t slot, const char* what) {
    g_err_slot = slot;
    snprintf(g_err, sizeof g_err, "buffer slot out of range: %u (%s)", slot, what);
    return HOLO_ERR_SLOT_OUT_OF_RANGE;
}
int32_t holo_cuda_fail(cudaError_t e, const char* where) {
    snprintf(g_err, sizeof g_err, "dispatch failed: CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), where);
    return HOLO_ERR_DISPATCH;
}

extern "C" const char* holo_b200_last_error(void) { return g_err; }
extern "C" uint32_t holo_b200_last_error_slot(void) { return g_err_slot; }
extern "C" const char* holo_b200_version(void) { return "hologram-b200 0.1 (sm_100a)"; }

// ---- context --------------------------------------------------------------------------------
extern "C" int32_t holo_b200_ctx_create(int32_t device, holo_b200_ctx** out) {
    if (!out) return holo_fail(HOLO_ERR_INIT, "backend init failed: null out pointer");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return holo_fail(HOLO_ERR_INIT, "backend init failed: no CUDA device (%s)", cudaGetErrorString(e));
    if (device < 0 || device >= count) return holo_fail(HOLO_ERR_INIT, "backend init failed: device %d of %d", device, count);
    if (cudaSetDevice(device) != cudaSuccess) return holo_fail(HOLO_ERR_INIT, "backend init failed: cudaSetDevice");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess)
        return holo_fail(HOLO_ERR_INIT, "backend init failed: cudaGetDeviceProperties");
    if (prop.major != 10)
        return holo_fail(HOLO_ERR_INIT, "backend init failed: device is sm_%d%d, this library is built for sm_100a only",
                         prop.major, prop.minor);
    holo_b200_ctx* ctx = new holo_b200_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return holo_fail(HOLO_ERR_INIT, "backend init failed: cudaStreamCreate");
    }
    ctx->own_stream = true;
    if (const char* e = getenv("HOLO_PDL")) ctx->pdl = atoi(e) != 0;
    if (cudaMalloc(&ctx->dev_status, 256) != cudaSuccess || cudaMemset(ctx->dev_status, 0, 256) != cudaSuccess) {
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return holo_fail(HOLO_ERR_INIT, "backend init failed: status word allocation");
    }
    if (cudaMalloc(&ctx->attn_arrivals, 65536 * 4) != cudaSuccess || cudaMemset(ctx->attn_arrivals, 0, 65536 * 4) != cudaSuccess) {
        cudaFree(ctx->dev_status);
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return holo_fail(HOLO_ERR_INIT, "backend init failed: arrival counter allocation");
    }
    cudaDeviceSynchronize();   // the clears above ran on the default stream, which the context's stream does not wait for
    *out = ctx;
    return HOLO_OK;
}

extern "C" void holo_b200_ctx_destroy(holo_b200_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    holo_tp_destroy(ctx);
    for (auto& row : ctx->lut)
        for (auto& t : row)
            if (t) cudaFree(t);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->stage) cudaFree(ctx->stage);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->attn_arrivals) cudaFree(ctx->attn_arrivals);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

extern "C" void* holo_b200_ctx_stream(holo_b200_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

extern "C" int32_t holo_b200_ctx_set_stream(holo_b200_ctx* ctx, void* stream) {
    if (!ctx) return holo_fail(HOLO_ERR_INIT, "null context");
    HOLO_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    ctx->stream = (cudaStream_t)stream;
    ctx->own_stream = false;
    return HOLO_OK;
}

// Asynchronous device-side failures (an out-of-range gather index, a bounded wait that gave
// up) are recorded in a status word and surface at the next synchronising call.
static int32_t check_dev_status(holo_b200_ctx* ctx) {
    uint32_t st = 0;
    HOLO_CUDA(cudaMemcpyAsync(&st, ctx->dev_status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    HOLO_CUDA(cudaStreamSynchronize(ctx->stream));
    if (st == 0) return HOLO_OK;
    cudaMemsetAsync(ctx->dev_status, 0, 4, ctx->stream);
    if (st & 2u) cudaMemsetAsync(ctx->attn_arrivals, 0, 65536 * 4, ctx->stream);  // a launch that gave up may have left counts behind
    if (st & 1u) return holo_fail_slot(HOLO_NO_SLOT, "gather index outside [−axis_dim, axis_dim)");
    return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: a device-side bounded wait gave up (status 0x%x)", st);
}

extern "C" int32_t holo_b200_ctx_synchronize(holo_b200_ctx* ctx) {
    if (!ctx) return holo_fail(HOLO_ERR_INIT, "null context");
    return check_dev_status(ctx);
}

extern "C" uint64_t holo_b200_ctx_launch_count(holo_b200_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int32_t holo_b200_ctx_set_lut_table(holo_b200_ctx* ctx, uint8_t act, uint8_t dtype, const uint16_t* table) {
    if (!ctx || !table) return holo_fail(HOLO_ERR_INIT, "null argument");
    const uint16_t* dev = nullptr;
    HOLO_TRY(holo_lut_table(ctx, act, dtype, &dev));
    HOLO_CUDA(cudaMemcpyAsync((void*)dev, table, 65536 * 2, cudaMemcpyHostToDevice, ctx->stream));
    HOLO_CUDA(cudaStreamSynchronize(ctx->stream));
    return HOLO_OK;
}

extern "C" int32_t holo_b200_ctx_get_lut_table(holo_b200_ctx* ctx, uint8_t act, uint8_t dtype, uint16_t* table) {
    if (!ctx || !table) return holo_fail(HOLO_ERR_INIT, "null argument");
    const uint16_t* dev = nullptr;
    HOLO_TRY(holo_lut_table(ctx, act, dtype, &dev));
    HOLO_CUDA(cudaMemcpyAsync(table, dev, 65536 * 2, cudaMemcpyDeviceToHost, ctx->stream));
    HOLO_CUDA(cudaStreamSynchronize(ctx->stream));
    return HOLO_OK;
}

int32_t holo_ensure_scratch(holo_b200_ctx* ctx, uint64_t bytes) {
    if (bytes <= ctx->scratch_bytes) return HOLO_OK;
    HOLO_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) cudaFree(ctx->scratch);
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    uint64_t want = (bytes + (1u << 20) - 1) & ~((uint64_t)(1u << 20) - 1);
    HOLO_CUDA(cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
    return HOLO_OK;
}

// ---- workspace ------------------------------------------------------------------------------
extern "C" int32_t holo_b200_workspace_create(holo_b200_ctx* ctx, uint32_t n_slots, holo_b200_workspace** out) {
    if (!ctx || !out) return holo_fail(HOLO_ERR_INIT, "null argument");
    auto* ws = new holo_b200_workspace();
    ws->ctx = ctx;
    ws->slots.resize(n_slots);
    *out = ws;
    return HOLO_OK;
}

extern "C" void holo_b200_workspace_destroy(holo_b200_workspace* ws) {
    if (!ws) return;
    cudaSetDevice(ws->ctx->device);
    cudaStreamSynchronize(ws->ctx->stream);
    for (auto& s : ws->slots)
        if (s.owned && s.ptr) cudaFree(s.ptr);
    delete ws;
}

extern "C" int32_t holo_b200_workspace_alloc(holo_b200_workspace* ws, uint32_t slot, uint64_t bytes) {
    if (!ws) return holo_fail(HOLO_ERR_INIT, "null workspace");
    if (slot >= ws->slots.size()) return holo_fail_slot(slot, "alloc");
    HoloSlot& s = ws->slots[slot];
    // 64-byte size granularity like the arena (crates/hologram-exec/src/buffer.rs:63).
    uint64_t cap = bytes ? ((bytes + 63) & ~63ull) : 64;
    if (!(s.owned && s.ptr && s.bytes == bytes)) {
        if (s.owned && s.ptr) {
            HOLO_CUDA(cudaStreamSynchronize(ws->ctx->stream));
            cudaFree(s.ptr);
        }
        s = HoloSlot();
        HOLO_CUDA(cudaMalloc(&s.ptr, cap));
        s.bytes = bytes;
        s.owned = true;
    }
    HOLO_CUDA(cudaMemsetAsync(s.ptr, 0, cap, ws->ctx->stream));
    return HOLO_OK;
}

extern "C" int32_t holo_b200_workspace_bind(holo_b200_workspace* ws, uint32_t slot, void* device_ptr, uint64_t bytes) {
    if (!ws) return holo_fail(HOLO_ERR_INIT, "null workspace");
    if (slot >= ws->slots.size()) return holo_fail_slot(slot, "bind");
    HoloSlot& s = ws->slots[slot];
    if (s.owned && s.ptr) {
        HOLO_CUDA(cudaStreamSynchronize(ws->ctx->stream));
        cudaFree(s.ptr);
    }
    s.ptr = device_ptr;
    s.bytes = bytes;
    s.owned = false;
    s.constant = false;
    return HOLO_OK;
}

extern "C" int32_t holo_b200_workspace_slot(holo_b200_workspace* ws, uint32_t slot, void** device_ptr, uint64_t* bytes) {
    if (!ws) return holo_fail(HOLO_ERR_INIT, "null workspace");
    if (slot >= ws->slots.size() || !ws->slots[slot].ptr) return holo_fail_slot(slot, "unbound");
    if (device_ptr) *device_ptr = ws->slots[slot].ptr;
    if (bytes) *bytes = ws->slots[slot].bytes;
    return HOLO_OK;
}

int32_t holo_resolve(holo_b200_workspace* ws, HoloBufferRef ref, uint64_t need, uint8_t** ptr, uint64_t* extent) {
    if (ref.slot >= ws->slots.size()) return holo_fail_slot(ref.slot, "no such slot");
    const HoloSlot& s = ws->slots[ref.slot];
    if (!s.ptr) return holo_fail_slot(ref.slot, "slot is not bound");
    if (ref.offset > s.bytes) return holo_fail_slot(ref.slot, "offset beyond slot");
    uint64_t ext = ref.length ? ref.length : s.bytes - ref.offset;
    if (ext > s.bytes - ref.offset) return holo_fail_slot(ref.slot, "range beyond slot");
    if (need > ext) return holo_fail_slot(ref.slot, "buffer shorter than the call's geometry requires");
    *ptr = (uint8_t*)s.ptr + ref.offset;
    if (extent) *extent = ext;
    return HOLO_OK;
}

extern "C" int32_t holo_b200_workspace_upload(holo_b200_workspace* ws, HoloBufferRef dst, const void* host, uint64_t bytes) {
    if (!ws) return holo_fail(HOLO_ERR_INIT, "null workspace");
    uint8_t* p;
    HOLO_TRY(holo_resolve(ws, dst, bytes, &p, nullptr));
    if (bytes) HOLO_CUDA(cudaMemcpyAsync(p, host, bytes, cudaMemcpyHostToDevice, ws->ctx->stream));
    return HOLO_OK;
}

extern "C" int32_t holo_b200_workspace_download(holo_b200_workspace* ws, HoloBufferRef src, void* host, uint64_t bytes) {
    if (!ws) return holo_fail(HOLO_ERR_INIT, "null workspace");
    uint8_t* p;
    HOLO_TRY(holo_resolve(ws, src, bytes, &p, nullptr));
    if (bytes) HOLO_CUDA(cudaMemcpyAsync(host, p, bytes, cudaMemcpyDeviceToHost, ws->ctx->stream));
    return check_dev_status(ws->ctx);
}

// ---- dispatch -------------------------------------------------------------------------------
namespace {

struct Range {
    const uint8_t* p;
    uint64_t n;
};
// split_borrow rule (workspace.rs:43-55, buffer.rs:955-999): the written range must not
// overlap any read range; the reference reports the failure against the output slot.
int32_t check_disjoint(const Range& w, uint32_t out_slot, std::initializer_list<Range> reads) {
    for (const Range& r : reads) {
        if (r.n == 0 || w.n == 0) continue;
        if (r.p < w.p + w.n && w.p < r.p + r.n) return holo_fail_slot(out_slot, "output overlaps an input range");
    }
    return HOLO_OK;
}

int lut_act_of_kind(uint16_t kind) {
    switch (kind) {
        case HOLO_K_SIGMOID: return HOLO_LUT_SIGMOID;
        case HOLO_K_TANH: return HOLO_LUT_TANH;
        case HOLO_K_GELU: return HOLO_LUT_GELU;
        case HOLO_K_SILU: return HOLO_LUT_SILU;
        case HOLO_K_EXP: return HOLO_LUT_EXP;
        case HOLO_K_ERF: return HOLO_LUT_ERF;
        default: return -1;
    }
}

// unary_act -> lut::unary_lut (cpu/kernels.rs:1586-1598, cpu/lut.rs:76-98)
int32_t do_unary_lut(holo_b200_ctx* ctx, const HoloUnaryCall& c, int act, holo_b200_workspace* ws) {
    if (c.dtype == HOLO_DTYPE_F64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: f64 is not a supported compute dtype (hologram computes in f16/bf16/f32)");
    if (c.dtype != HOLO_DTYPE_F16 && c.dtype != HOLO_DTYPE_BF16)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: this backend serves unary activations through the 16-bit LUT only (dtype %u)", c.dtype);
    uint64_t n = c.element_count;
    if (n == 0) return HOLO_OK;
    uint8_t *in, *out;
    // the reference resolves the borrow first (output slot reported), then the lengths
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.input, n * 2, &in, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, n * 2, &out, nullptr));
    HOLO_TRY(check_disjoint({out, n * 2}, c.output.slot, {{in, n * 2}}));
    const uint16_t* table;
    HOLO_TRY(holo_lut_table(ctx, (uint8_t)act, c.dtype, &table));
    return holo_launch_lut(ctx, table, (const uint16_t*)in, (uint16_t*)out, n);
}

// binary_float_acc (cpu/float_kernels.rs:252-296)
int32_t do_binary(holo_b200_ctx* ctx, const HoloBinaryCall& c, int op, holo_b200_workspace* ws) {
    if (c.dtype == HOLO_DTYPE_F64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: f64 is not a supported compute dtype (hologram computes in f16/bf16/f32)");
    if (!holo_is_compute_float(c.dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: integer-ring Add/Mul are not served by this backend (dtype %u)", c.dtype);
    uint64_t bytes = c.element_count * holo_dtype_size(c.dtype);
    uint8_t *a, *b, *out;
    HOLO_TRY(holo_resolve(ws, c.a, bytes, &a, nullptr));
    HOLO_TRY(holo_resolve(ws, c.b, bytes, &b, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, bytes, &out, nullptr));
    HOLO_TRY(check_disjoint({out, bytes}, c.a.slot, {{a, bytes}, {b, bytes}}));
    return holo_launch_binary(ctx, op, a, b, out, c.element_count, c.dtype);
}

// unary_float / binary_float with an exact IEEE operation (cpu/float_kernels.rs:190-233, :236-296)
int32_t do_elementwise(holo_b200_ctx* ctx, const HoloKernelCall* call, holo_b200_workspace* ws) {
    const bool unary = holo_is_exact_unary(call->kind);
    const uint8_t dtype = unary ? call->u.unary.dtype : call->u.binary.dtype;
    const uint64_t n = unary ? call->u.unary.element_count : call->u.binary.element_count;
    if (dtype == HOLO_DTYPE_F64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: f64 is not a supported compute dtype (hologram computes in f16/bf16/f32)");
    if (!holo_is_compute_float(dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: the integer-ring form of variant %u is not served by this backend (dtype %u)", call->kind, dtype);
    if (n == 0) return HOLO_OK;
    const uint64_t bytes = n * holo_dtype_size(dtype);
    uint8_t *a, *b = nullptr, *out;
    if (unary) {
        HOLO_TRY(holo_resolve(ws, call->u.unary.output, 0, &out, nullptr));
        HOLO_TRY(holo_resolve(ws, call->u.unary.input, bytes, &a, nullptr));
        HOLO_TRY(holo_resolve(ws, call->u.unary.output, bytes, &out, nullptr));
        HOLO_TRY(check_disjoint({out, bytes}, call->u.unary.output.slot, {{a, bytes}}));
    } else {
        HOLO_TRY(holo_resolve(ws, call->u.binary.a, bytes, &a, nullptr));
        HOLO_TRY(holo_resolve(ws, call->u.binary.b, bytes, &b, nullptr));
        HOLO_TRY(holo_resolve(ws, call->u.binary.output, bytes, &out, nullptr));
        HOLO_TRY(check_disjoint({out, bytes}, call->u.binary.a.slot, {{a, bytes}, {b, bytes}}));
    }
    return holo_launch_elementwise(ctx, (int)call->kind, a, b, out, n, dtype);
}

// matmul_float and its fused epilogues (cpu/float_kernels.rs:298-399, 822-891)
int32_t do_matmul(holo_b200_ctx* ctx, const HoloMatMulCall& c, uint8_t act, const HoloBufferRef* residual,
                  holo_b200_workspace* ws) {
    if (c.m == 0 || c.k == 0 || c.n == 0) return HOLO_OK;
    if (c.dtype == HOLO_DTYPE_F64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: f64 is not a supported compute dtype (hologram computes in f16/bf16/f32)");
    if (!holo_is_compute_float(c.dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul: only f32/f16/bf16 are supported compute dtypes (dtype %u)", c.dtype);
    if (c.b_packed) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: panel-packed B is an f32-only layout");
    if (act != 0 && act != HOLO_FUSED_GELU && act != HOLO_FUSED_SILU && act != HOLO_FUSED_SIGMOID && act != HOLO_FUSED_TANH &&
        act != HOLO_FUSED_EXP)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: fused activation %u is not table-backed", act);
    const uint64_t es = holo_dtype_size(c.dtype);
    uint64_t ab = (uint64_t)c.m * c.k * es, bb = (uint64_t)c.k * c.n * es, ob = (uint64_t)c.m * c.n * es;
    uint8_t *a, *b, *out, *res = nullptr;
    HOLO_TRY(holo_resolve(ws, c.a, ab, &a, nullptr));
    HOLO_TRY(holo_resolve(ws, c.b, bb, &b, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, ob, &out, nullptr));
    HOLO_TRY(check_disjoint({out, ob}, c.a.slot, {{a, ab}, {b, bb}}));
    if (residual) {
        HOLO_TRY(holo_resolve(ws, *residual, ob, &res, nullptr));
        HOLO_TRY(check_disjoint({out, ob}, c.output.slot, {{res, ob}}));
    }
    const bool b_constant = c.b.slot < ws->slots.size() && ws->slots[c.b.slot].constant;
    return holo_launch_matmul(ctx, a, b, out, c.m, c.k, c.n, c.dtype, act, res, b_constant);
}

// matmul_add_activation_float (cpu/float_kernels.rs:899-938): act(A . B + residual), served on the exact per-cell kernel
int32_t do_matmul_add_activation(holo_b200_ctx* ctx, const HoloMatMulAddActivationCall& c, holo_b200_workspace* ws) {
    const HoloMatMulCall& mm = c.mm;
    if (mm.m == 0 || mm.k == 0 || mm.n == 0) return HOLO_OK;
    if (mm.dtype == HOLO_DTYPE_F64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: f64 is not a supported compute dtype (hologram computes in f16/bf16/f32)");
    if (!holo_is_compute_float(mm.dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul: only f32/f16/bf16 are supported compute dtypes (dtype %u)", mm.dtype);
    if (mm.b_packed) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: panel-packed B is not served by this backend");
    if (c.act != HOLO_FUSED_GELU && c.act != HOLO_FUSED_SILU && c.act != HOLO_FUSED_SIGMOID && c.act != HOLO_FUSED_TANH && c.act != HOLO_FUSED_EXP)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_add_activation: fused activation %u is not served", c.act);
    const uint64_t es = holo_dtype_size(mm.dtype);
    const uint64_t ab = (uint64_t)mm.m * mm.k * es, bb = (uint64_t)mm.k * mm.n * es, ob = (uint64_t)mm.m * mm.n * es;
    uint8_t *a, *b, *out, *res;
    HOLO_TRY(holo_resolve(ws, mm.a, ab, &a, nullptr));
    HOLO_TRY(holo_resolve(ws, mm.b, bb, &b, nullptr));
    HOLO_TRY(holo_resolve(ws, mm.output, ob, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.residual, ob, &res, nullptr));
    HOLO_TRY(check_disjoint({out, ob}, mm.output.slot, {{a, ab}, {b, bb}, {res, ob}}));
    return holo_launch_matmul_add_activation(ctx, a, b, out, mm.m, mm.k, mm.n, mm.dtype, c.act, res);
}

// matmul_dequant_float over a [k, n] weight with f32 activations (cpu/float_kernels.rs:596-731) + epilogue (:733-770)
int32_t do_matmul_dequant_kn(holo_b200_ctx* ctx, const HoloMatMulDequantCall& c, holo_b200_workspace* ws) {
    const bool per_channel = c.channels > 0 && c.scales.slot != HOLO_NO_SLOT;
    if (c.codebook.slot != HOLO_NO_SLOT || c.quant_dtype == HOLO_DTYPE_E8CB)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: quant_dtype is not scalar-decodable (e8cb needs its codebook operand and the fused omajor path)");
    if (c.quant_dtype != HOLO_DTYPE_I8 && c.quant_dtype != HOLO_DTYPE_U8 && c.quant_dtype != HOLO_DTYPE_I4)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: unknown quantized weight tier");
    int act = -1;
    if (c.act != 0) {
        if (c.act != HOLO_FUSED_GELU && c.act != HOLO_FUSED_SILU && c.act != HOLO_FUSED_SIGMOID && c.act != HOLO_FUSED_TANH && c.act != HOLO_FUSED_EXP)
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: fused activation %u is not served", c.act);
        act = c.act == HOLO_FUSED_GELU ? HOLO_LUT_GELU : c.act == HOLO_FUSED_SILU ? HOLO_LUT_SILU : c.act == HOLO_FUSED_SIGMOID ? HOLO_LUT_SIGMOID
              : c.act == HOLO_FUSED_TANH ? HOLO_LUT_TANH : HOLO_LUT_EXP;
    }
    const uint64_t kn = (uint64_t)c.k * c.n;
    const uint64_t ab = (uint64_t)c.m * c.k * 4, wb = c.quant_dtype == HOLO_DTYPE_I4 ? (kn + 1) / 2 : kn, sb = (uint64_t)c.channels * 4, ob = (uint64_t)c.m * c.n * 4;
    uint8_t *a, *bq, *sc = nullptr, *zp = nullptr, *res = nullptr, *out;
    HOLO_TRY(holo_resolve(ws, c.output, ob, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.a, ab, &a, nullptr));
    HOLO_TRY(holo_resolve(ws, c.bq, wb, &bq, nullptr));
    if (per_channel) {
        HOLO_TRY(holo_resolve(ws, c.scales, sb, &sc, nullptr));
        HOLO_TRY(holo_resolve(ws, c.zero_points, sb, &zp, nullptr));
    }
    if (c.residual.slot != HOLO_NO_SLOT) HOLO_TRY(holo_resolve(ws, c.residual, ob, &res, nullptr));
    HOLO_TRY(check_disjoint({out, ob}, c.output.slot, {{a, ab}, {bq, wb}, {sc, sc ? sb : 0}, {zp, zp ? sb : 0}, {res, res ? ob : 0}}));
    if ((((uintptr_t)a | (uintptr_t)sc | (uintptr_t)zp | (uintptr_t)res | (uintptr_t)out) & 3u) != 0)
        return holo_fail_slot(c.a.slot, "matmul_dequant f32 operands must be 4-byte aligned on the device");
    float scale;
    memcpy(&scale, &c.scale_bits, 4);
    return holo_launch_matmul_dequant_kn(ctx, (const float*)a, bq, (const float*)sc, (const int32_t*)zp, (const float*)res, (float*)out, c.m, c.k, c.n,
                                         c.channels, c.inner, c.quant_dtype, scale, c.zero_point, act);
}

// matmul_dequant_float, the output-major W8A8 arm (cpu/float_kernels.rs:534-596) + epilogue (:727-766)
int32_t do_matmul_dequant(holo_b200_ctx* ctx, const HoloMatMulDequantCall& c, holo_b200_workspace* ws) {
    if (c.m == 0 || c.k == 0 || c.n == 0) return HOLO_OK;
    if (c.dtype != HOLO_DTYPE_F32) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: only f32 output is supported");
    if (!c.bq_omajor || c.act_quant != 1) {
        // an output-major weight must never be read with the [k,n] interpretation, and W8A8 has one emitter (float_kernels.rs:534-553)
        if (c.bq_omajor || c.act_quant != 0)
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: bq_omajor and W8A8 must be paired");
        return do_matmul_dequant_kn(ctx, c, ws);
    }
    const bool per_channel = c.channels > 0 && c.scales.slot != HOLO_NO_SLOT;
    const bool i4 = c.quant_dtype == HOLO_DTYPE_I4, e8 = c.quant_dtype == HOLO_DTYPE_E8CB;
    if (e8 != (c.codebook.slot != HOLO_NO_SLOT))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: a codebook operand goes with the E8 codebook weight tier and only with it");
    if (e8 && (c.k & 7u))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: k must be a multiple of 8 (whole E8 groups)");
    if ((c.quant_dtype != HOLO_DTYPE_I8 && !i4 && !e8) || !per_channel || c.channels != c.n || c.inner != 1 || c.k > 133144u || (i4 && (c.k & 1u)))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: W8A8 requires symmetric per-channel i8/i4/e8cb within the k bound (all three are served)");
    int act = -1;
    if (c.act != 0) {
        if (c.act != HOLO_FUSED_GELU && c.act != HOLO_FUSED_SILU && c.act != HOLO_FUSED_SIGMOID && c.act != HOLO_FUSED_TANH && c.act != HOLO_FUSED_EXP)
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: matmul_dequant: fused activation %u is not served", c.act);
        act = c.act == HOLO_FUSED_GELU ? HOLO_LUT_GELU : c.act == HOLO_FUSED_SILU ? HOLO_LUT_SILU : c.act == HOLO_FUSED_SIGMOID ? HOLO_LUT_SIGMOID
              : c.act == HOLO_FUSED_TANH ? HOLO_LUT_TANH : HOLO_LUT_EXP;
    }
    const uint64_t ab = (uint64_t)c.m * c.k * 4, wb = e8 ? (uint64_t)c.n * (c.k / 8) : i4 ? (uint64_t)c.n * (c.k / 2) : (uint64_t)c.n * c.k, sb = (uint64_t)c.n * 4, ob = (uint64_t)c.m * c.n * 4;
    uint8_t *a, *bq, *sc, *zp = nullptr, *res = nullptr, *out, *cb = nullptr;
    HOLO_TRY(holo_resolve(ws, c.output, ob, &out, nullptr));
    if (e8) HOLO_TRY(holo_resolve(ws, c.codebook, 2048, &cb, nullptr));   // the full index space: 256 entries x 8 coordinates
    HOLO_TRY(holo_resolve(ws, c.a, ab, &a, nullptr));
    HOLO_TRY(holo_resolve(ws, c.bq, wb, &bq, nullptr));
    HOLO_TRY(holo_resolve(ws, c.scales, sb, &sc, nullptr));
    if (c.zero_points.slot != HOLO_NO_SLOT) HOLO_TRY(holo_resolve(ws, c.zero_points, sb, &zp, nullptr));
    if (c.residual.slot != HOLO_NO_SLOT) HOLO_TRY(holo_resolve(ws, c.residual, ob, &res, nullptr));
    HOLO_TRY(check_disjoint({out, ob}, c.output.slot, {{a, ab}, {bq, wb}, {sc, sb}, {zp, zp ? sb : 0}, {res, res ? ob : 0}}));
    if ((((uintptr_t)a | (uintptr_t)sc | (uintptr_t)zp | (uintptr_t)res | (uintptr_t)out) & 3u) != 0)
        return holo_fail_slot(c.a.slot, "matmul_dequant f32 operands must be 4-byte aligned on the device");
    if (e8)
        return holo_launch_matmul_e8cb_omajor(ctx, (const float*)a, bq, (const int8_t*)cb, (const float*)sc, (const int32_t*)zp, (const float*)res,
                                              (float*)out, c.m, c.k, c.n, act);
    return holo_launch_matmul_w8a8_omajor(ctx, (const float*)a, (const int8_t*)bq, (const float*)sc, (const int32_t*)zp, (const float*)res,
                                          (float*)out, c.m, c.k, c.n, act, i4);
}

// rms_norm_float (cpu/float_kernels.rs:1683-1756), epsilon rule :1324-1336
// `with_residual`: add_rms_norm_float (:1567-1681); an absent residual operand makes it a plain RmsNorm
int32_t do_norm(holo_b200_ctx* ctx, const HoloNormCall& c, bool with_residual, bool layer, holo_b200_workspace* ws) {
    if (c.batch == 0 || c.feature == 0) return HOLO_OK;
    if (!holo_is_compute_float(c.dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: %s dtype %u", layer ? "layer_norm" : "rms_norm", c.dtype);
    if (c.num_groups != 0) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: grouped norms are not served by this backend");
    float eps = 1e-9f;
    if (c.epsilon_bits != 0) {
        uint32_t b = (uint32_t)c.epsilon_bits;
        memcpy(&eps, &b, 4);
        if (!(isfinite(eps) && eps > 0.0f))
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: norm epsilon must be a positive finite f32 (0 selects the default)");
    }
    size_t es = holo_dtype_size(c.dtype);
    uint64_t total = (uint64_t)c.batch * c.feature * es, row = (uint64_t)c.feature * es;
    uint8_t *x, *g = nullptr, *beta = nullptr, *res = nullptr, *out;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.x, total, &x, nullptr));
    if (with_residual && c.residual.slot != HOLO_NO_SLOT) HOLO_TRY(holo_resolve(ws, c.residual, total, &res, nullptr));
    if (c.gamma.slot != HOLO_NO_SLOT) HOLO_TRY(holo_resolve(ws, c.gamma, row, &g, nullptr));
    if (layer && c.beta.slot != HOLO_NO_SLOT) HOLO_TRY(holo_resolve(ws, c.beta, row, &beta, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, total, &out, nullptr));
    HOLO_TRY(check_disjoint({out, total}, c.output.slot, {{x, total}, {res, res ? total : 0}, {g, g ? row : 0}, {beta, beta ? row : 0}}));
    if (layer) return holo_launch_layer_norm(ctx, x, g, beta, out, c.batch, c.feature, eps, c.dtype);   // layer_norm_float (cpu/float_kernels.rs:1338-1445)
    return holo_launch_rms_norm(ctx, x, res, g, out, c.batch, c.feature, eps, c.dtype);
}

// softmax_float (cpu/float_kernels.rs:1758-1875)
int32_t do_softmax(holo_b200_ctx* ctx, const HoloSoftmaxCall& c, holo_b200_workspace* ws) {
    if (c.batch == 0 || c.feature == 0) return HOLO_OK;
    if (!holo_is_compute_float(c.dtype)) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: softmax dtype %u", c.dtype);
    const uint64_t total = (uint64_t)c.batch * c.feature * holo_dtype_size(c.dtype);
    uint8_t *x, *out;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.input, total, &x, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, total, &out, nullptr));
    HOLO_TRY(check_disjoint({out, total}, c.output.slot, {{x, total}}));
    return holo_launch_softmax(ctx, x, out, c.batch, c.feature, c.dtype);
}

// rope_float (cpu/float_kernels.rs:3123-3190)
int32_t do_rope(holo_b200_ctx* ctx, const HoloRoPECall& c, holo_b200_workspace* ws) {
    uint64_t n = c.element_count;
    uint32_t d = c.head_dim;
    if (d == 0 || d % 2 != 0 || n % d != 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: rope: head_dim must be even and divide the element count");
    if (!holo_is_compute_float(c.dtype)) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: rope dtype %u", c.dtype);
    uint64_t bytes = n * holo_dtype_size(c.dtype);
    uint8_t *x, *cs, *sn, *out;
    HOLO_TRY(holo_resolve(ws, c.output, bytes, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.x, bytes, &x, nullptr));
    HOLO_TRY(holo_resolve(ws, c.cos, bytes, &cs, nullptr));
    HOLO_TRY(holo_resolve(ws, c.sin, bytes, &sn, nullptr));
    HOLO_TRY(check_disjoint({out, bytes}, c.output.slot, {{x, bytes}, {cs, bytes}, {sn, bytes}}));
    return holo_launch_rope(ctx, x, cs, sn, out, d, n, c.dtype);
}

// gather (cpu/kernels.rs:389-446)
int32_t do_gather(holo_b200_ctx* ctx, const HoloGatherCall& c, holo_b200_workspace* ws) {
    size_t es = holo_dtype_size(c.dtype);
    if (es == 0) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: gather: sub-byte or unknown element dtype not supported");
    size_t iw = c.idx_dtype == HOLO_DTYPE_I32 ? 4 : c.idx_dtype == HOLO_DTYPE_I64 ? 8 : 0;
    if (iw == 0) return holo_fail_slot(c.indices.slot, "gather index dtype must be i32 or i64");
    uint64_t row = c.inner * es;
    uint8_t *data, *idx, *out;
    uint64_t db = c.outer * c.axis_dim * row, ib = c.num_indices * iw, ob = c.outer * c.num_indices * row;
    if (holo_resolve(ws, c.data, db, &data, nullptr) != HOLO_OK || holo_resolve(ws, c.indices, ib, &idx, nullptr) != HOLO_OK ||
        holo_resolve(ws, c.output, ob, &out, nullptr) != HOLO_OK)
        return holo_fail_slot(c.output.slot, "gather operand shorter than its geometry");
    HOLO_TRY(check_disjoint({out, ob}, c.output.slot, {{data, db}, {idx, ib}}));
    return holo_launch_gather(ctx, data, idx, c.idx_dtype, out, c.outer, c.axis_dim, row, c.num_indices);
}

// cast (cpu/kernels.rs:560-594)
int32_t do_cast(holo_b200_ctx* ctx, const HoloCastCall& c, holo_b200_workspace* ws) {
    size_t sw = holo_dtype_size(c.src_dtype), dw = holo_dtype_size(c.dst_dtype);
    if (sw == 0 || dw == 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: cast: unsupported source/destination dtype (sub-byte not castable)");
    if (c.dst_dtype == HOLO_DTYPE_F64 || c.dst_dtype == HOLO_DTYPE_U64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: cast to dtype %u is not served by this backend", c.dst_dtype);
    uint8_t *in, *out;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.input, c.element_count * sw, &in, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, c.element_count * dw, &out, nullptr));
    HOLO_TRY(check_disjoint({out, c.element_count * dw}, c.output.slot, {{in, c.element_count * sw}}));
    return holo_launch_cast(ctx, in, c.src_dtype, out, c.dst_dtype, c.element_count);
}

// Reshape dispatched as a call is a byte copy (the executor normally label-propagates it,
// crates/hologram-exec/src/session.rs:1112-1114).
int32_t do_reshape(holo_b200_ctx* ctx, const HoloLayoutCall& c, holo_b200_workspace* ws) {
    size_t es = holo_dtype_size(c.dtype);
    if (es == 0) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: reshape of a sub-byte dtype");
    uint64_t bytes = c.element_count * es;
    uint8_t *in, *out;
    HOLO_TRY(holo_resolve(ws, c.input, bytes, &in, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, bytes, &out, nullptr));
    HOLO_TRY(check_disjoint({out, bytes}, c.output.slot, {{in, bytes}}));
    if (bytes) HOLO_CUDA(cudaMemcpyAsync(out, in, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return HOLO_OK;
}

// concat_float (cpu/float_kernels.rs:2963-2974): out = a || b, both taken at their resolved
// extents; dtype-agnostic byte placement.
int32_t do_concat(holo_b200_ctx* ctx, const HoloBinaryCall& c, holo_b200_workspace* ws) {
    uint8_t *a, *b, *out;
    uint64_t alen = 0, blen = 0, olen = 0;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, &olen));
    HOLO_TRY(holo_resolve(ws, c.a, 0, &a, &alen));
    HOLO_TRY(holo_resolve(ws, c.b, 0, &b, &blen));
    if (olen < alen + blen) return holo_fail_slot(c.output.slot, "concat output shorter than a || b");
    HOLO_TRY(check_disjoint({out, alen + blen}, c.output.slot, {{a, alen}, {b, blen}}));
    if (alen) HOLO_CUDA(cudaMemcpyAsync(out, a, alen, cudaMemcpyDeviceToDevice, ctx->stream));
    if (blen) HOLO_CUDA(cudaMemcpyAsync(out + alen, b, blen, cudaMemcpyDeviceToDevice, ctx->stream));
    return HOLO_OK;
}

// transpose_float (cpu/float_kernels.rs:2980-3027)
int32_t do_transpose(holo_b200_ctx* ctx, const HoloTransposeCall& c, holo_b200_workspace* ws) {
    if (c.rank == 0 || c.rank > 8) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: transpose: rank must be 1..=8");
    size_t es = holo_dtype_size(c.dtype);
    if (es == 0) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: transpose of a sub-byte dtype");
    uint64_t total = 1;
    uint32_t seen = 0;
    for (uint32_t i = 0; i < c.rank; ++i) {
        total *= c.dims[i];
        if (c.perm[i] >= c.rank || (seen & (1u << c.perm[i]))) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: transpose: perm is not a permutation of the axes");
        seen |= 1u << c.perm[i];
    }
    uint8_t *in, *out;
    HOLO_TRY(holo_resolve(ws, c.output, total * es, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.input, total * es, &in, nullptr));
    HOLO_TRY(check_disjoint({out, total * es}, c.output.slot, {{in, total * es}}));
    if (((uintptr_t)in | (uintptr_t)out) % es != 0) return holo_fail_slot(c.input.slot, "transpose operands must be aligned to the element size on the device");
    return holo_launch_transpose(ctx, in, out, c.rank, c.dims, c.perm, (uint32_t)es);
}

// expand_float / broadcast_binary_float (cpu/float_kernels.rs:3405-3444, :3250-3397). `other` null = Expand.
int32_t do_broadcast(holo_b200_ctx* ctx, const char* name, HoloBufferRef small_ref, const HoloBufferRef* other_ref, HoloBufferRef out_ref,
                     uint8_t rank, const uint32_t* in_dims, const uint32_t* out_dims, int op, int small_is_lhs, uint8_t dtype,
                     holo_b200_workspace* ws) {
    if (rank == 0 || rank > 8) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: %s: rank must be 1..=8", name);
    const size_t es = holo_dtype_size(dtype);
    if (es == 0) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: %s of a sub-byte dtype", name);
    if (other_ref && !holo_is_compute_float(dtype)) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: %s dtype %u", name, dtype);
    if (other_ref && op > HOLO_BROADCAST_MUL) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: %s: bad op", name);
    uint64_t out_total = 1, small_total = 1;
    for (uint32_t i = 0; i < rank; ++i) {
        if (in_dims[i] != 1 && in_dims[i] != out_dims[i])
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: %s: axis %u has %u elements against %u (must be 1 or equal)", name, i, in_dims[i], out_dims[i]);
        out_total *= out_dims[i];
        small_total *= in_dims[i];
    }
    uint8_t *small, *other = nullptr, *out;
    HOLO_TRY(holo_resolve(ws, out_ref, out_total * es, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, small_ref, small_total * es, &small, nullptr));
    if (other_ref) HOLO_TRY(holo_resolve(ws, *other_ref, out_total * es, &other, nullptr));
    HOLO_TRY(check_disjoint({out, out_total * es}, out_ref.slot, {{small, small_total * es}, {other, other ? out_total * es : 0}}));
    if (((uintptr_t)small | (uintptr_t)out | (uintptr_t)other) % es != 0) return holo_fail_slot(small_ref.slot, "broadcast operands must be aligned to the element size on the device");
    return holo_launch_broadcast(ctx, small, other, out, rank, in_dims, out_dims, (uint32_t)es, other_ref ? op : -1, small_is_lhs, dtype);
}

// where_float (cpu/float_kernels.rs:2908-2937)
int32_t do_where(holo_b200_ctx* ctx, const HoloWhereCall& c, holo_b200_workspace* ws) {
    if (!holo_is_compute_float(c.dtype)) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: where dtype %u", c.dtype);
    const uint64_t n = c.element_count, bytes = n * holo_dtype_size(c.dtype);
    uint8_t *cond, *a, *b, *out;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.cond, n, &cond, nullptr));
    HOLO_TRY(holo_resolve(ws, c.a, bytes, &a, nullptr));
    HOLO_TRY(holo_resolve(ws, c.b, bytes, &b, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, bytes, &out, nullptr));
    HOLO_TRY(check_disjoint({out, bytes}, c.output.slot, {{cond, n}, {a, bytes}, {b, bytes}}));
    return holo_launch_where(ctx, cond, a, b, out, n, c.dtype);
}

// dequant_activation (cpu/kernels.rs:311-381)
int32_t do_dequant_activation(holo_b200_ctx* ctx, const HoloDequantActivationCall& c, holo_b200_workspace* ws) {
    const uint64_t n = c.element_count;
    if (c.quant_dtype != HOLO_DTYPE_I8 && c.quant_dtype != HOLO_DTYPE_U8 && c.quant_dtype != HOLO_DTYPE_I4)
        return holo_fail_slot(c.input.slot, "dequant_activation source must be i8, u8 or i4");
    if (c.dtype != HOLO_DTYPE_F32) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: dequant_activation writes f32 (dtype %u)", c.dtype);
    if (c.act >= HOLO_LUT_COUNT) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: dequant_activation: unknown activation id %u", c.act);
    const uint64_t in_bytes = c.quant_dtype == HOLO_DTYPE_I4 ? (n + 1) / 2 : n;
    uint8_t *in, *out;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.input, in_bytes, &in, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, n * 4, &out, nullptr));
    HOLO_TRY(check_disjoint({out, n * 4}, c.output.slot, {{in, in_bytes}}));
    if (((uintptr_t)out & 3u) != 0) return holo_fail_slot(c.output.slot, "dequant_activation output must be 4-byte aligned on the device");
    float scale;
    memcpy(&scale, &c.scale_bits, 4);
    return holo_launch_dequant_activation(ctx, in, (float*)out, n, c.quant_dtype, c.act, scale, c.zero_point);
}

// reduce_float (cpu/float_kernels.rs:1901-2022)
uint64_t reduce_out_count(const HoloReduceCall& c) {
    uint64_t out = 1;
    if (c.rank == 0 || c.axes_mask == 0) return 1;
    for (uint32_t i = 0; i < c.rank && i < 8; ++i)
        if (!((c.axes_mask >> i) & 1u)) out *= c.dims[i];
    return out;
}
int32_t do_reduce(holo_b200_ctx* ctx, const HoloReduceCall& c, int kind, int mean, holo_b200_workspace* ws) {
    const uint64_t n = c.element_count;
    if (n == 0) return HOLO_OK;
    if (!holo_is_compute_float(c.dtype)) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: reduce dtype %u", c.dtype);
    if (c.rank > 8) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: reduce: rank must be <= 8");
    if (n > 0xffffffffull && c.rank == 0) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: reduce: a rank-0 input above 2^32 elements");
    uint64_t prod = 1;
    for (uint32_t i = 0; i < c.rank; ++i) prod *= c.dims[i];
    if (c.rank > 0 && prod != n) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: reduce: dims product != element_count");
    const size_t es = holo_dtype_size(c.dtype);
    const uint64_t out_count = reduce_out_count(c);
    uint8_t *in, *out;
    HOLO_TRY(holo_resolve(ws, c.output, out_count * es, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.input, n * es, &in, nullptr));
    HOLO_TRY(check_disjoint({out, out_count * es}, c.output.slot, {{in, n * es}}));
    return holo_launch_reduce(ctx, in, out, c.rank, c.dims, c.axes_mask, n, kind, mean, c.dtype);
}

// dequantize (cpu/kernels.rs:185-296)
int32_t do_dequantize(holo_b200_ctx* ctx, const HoloDequantizeCall& c, holo_b200_workspace* ws) {
    if (c.quant_dtype != HOLO_DTYPE_I8 && c.quant_dtype != HOLO_DTYPE_U8) return holo_fail_slot(c.input.slot, "dequantize source must be i8 or u8");
    if (!holo_is_compute_float(c.dtype)) return holo_fail_slot(c.output.slot, "dequantize destination must be f32, bf16 or f16");
    uint64_t n = c.element_count;
    bool per_ch = c.channels > 0 && c.scales.slot != HOLO_NO_SLOT;
    uint8_t *in, *out, *sc = nullptr, *zp = nullptr;
    uint64_t ob = n * holo_dtype_size(c.dtype);
    HOLO_TRY(holo_resolve(ws, c.output, ob, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.input, n, &in, nullptr));
    if (per_ch) {
        HOLO_TRY(holo_resolve(ws, c.scales, (uint64_t)c.channels * 4, &sc, nullptr));
        if (c.zero_points.slot != HOLO_NO_SLOT) HOLO_TRY(holo_resolve(ws, c.zero_points, (uint64_t)c.channels * 4, &zp, nullptr));
        else return holo_fail_slot(c.zero_points.slot, "per-channel dequantize needs a zero-point vector");
    }
    HOLO_TRY(check_disjoint({out, ob}, c.output.slot, {{in, n}}));
    return holo_launch_dequantize(ctx, c, in, (const float*)sc, (const int32_t*)zp, out);
}

// kv_cache_write (cpu/kernels.rs:455-501)
int32_t do_kv_write(holo_b200_ctx* ctx, const HoloKvCacheWriteCall& c, holo_b200_workspace* ws) {
    if (c.bucket_rows == 0 || c.row_bytes == 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: kv_cache_write: bucket_rows and row_bytes must be >= 1");
    if (c.new_rows > c.bucket_rows)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: kv_cache_write: new_rows exceeds bucket_rows");
    uint64_t plane = (uint64_t)c.bucket_rows * c.row_bytes, total = plane * c.planes;
    uint64_t nb = (uint64_t)c.planes * c.new_rows * c.row_bytes;
    uint8_t *cache, *nw, *pos, *out;
    if (holo_resolve(ws, c.cache, total, &cache, nullptr) != HOLO_OK || holo_resolve(ws, c.new_rows_buf, nb, &nw, nullptr) != HOLO_OK ||
        holo_resolve(ws, c.pos, 4, &pos, nullptr) != HOLO_OK || holo_resolve(ws, c.output, total, &out, nullptr) != HOLO_OK)
        return holo_fail_slot(c.output.slot, "kv_cache_write operand shorter than its geometry");
    if (out == cache) {
        // in-place move form: only the new rows are written
        HOLO_TRY(check_disjoint({out, total}, c.output.slot, {{nw, nb}, {pos, 4}}));
    } else {
        HOLO_TRY(check_disjoint({out, total}, c.output.slot, {{cache, total}, {nw, nb}, {pos, 4}}));
    }
    if (((uintptr_t)pos & 3u) != 0) return holo_fail_slot(c.pos.slot, "pos operand must be 4-byte aligned on the device");
    return holo_launch_kv_write(ctx, cache, nw, (const uint32_t*)pos, out, c.planes, c.bucket_rows, c.new_rows, c.row_bytes);
}

int32_t do_quantize_rows(holo_b200_ctx* ctx, const HoloQuantizeRowsI8Call& c, holo_b200_workspace* ws) {
    if (!holo_is_compute_float(c.dtype)) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: quantize_rows_i8 input dtype %u", c.dtype);
    uint64_t n = c.rows * c.row_len;
    uint64_t ib = n * holo_dtype_size(c.dtype);
    uint8_t *in, *codes, *scales;
    HOLO_TRY(holo_resolve(ws, c.input, ib, &in, nullptr));
    HOLO_TRY(holo_resolve(ws, c.codes, n, &codes, nullptr));
    HOLO_TRY(holo_resolve(ws, c.scales, c.rows * 4, &scales, nullptr));
    HOLO_TRY(check_disjoint({codes, n}, c.codes.slot, {{in, ib}, {scales, c.rows * 4}}));
    HOLO_TRY(check_disjoint({scales, c.rows * 4}, c.scales.slot, {{in, ib}}));
    if (((uintptr_t)scales & 3u) != 0) return holo_fail_slot(c.scales.slot, "scales must be 4-byte aligned");
    return holo_launch_quantize_rows(ctx, in, c.dtype, c.rows, c.row_len, (int8_t*)codes, (float*)scales);
}

// Extension: RotaryEmbedding + QuantizeRowsI8 over the rotated rows (one row = one head).
int32_t do_rope_quantize(holo_b200_ctx* ctx, const HoloRopeQuantizeCall& c, holo_b200_workspace* ws) {
    if (!holo_is_compute_float(c.dtype)) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: rope_quantize_rows_i8 dtype %u", c.dtype);
    if (c.row_len == 0 || c.row_len % 2 != 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: rope: head_dim must be even and divide the element count");
    const uint64_t n = c.rows * c.row_len, ib = n * holo_dtype_size(c.dtype);
    uint8_t *x, *co, *si, *ro, *codes, *scales;
    HOLO_TRY(holo_resolve(ws, c.rope_output, ib, &ro, nullptr));
    HOLO_TRY(holo_resolve(ws, c.x, ib, &x, nullptr));
    HOLO_TRY(holo_resolve(ws, c.cos, ib, &co, nullptr));
    HOLO_TRY(holo_resolve(ws, c.sin, ib, &si, nullptr));
    HOLO_TRY(holo_resolve(ws, c.codes, n, &codes, nullptr));
    HOLO_TRY(holo_resolve(ws, c.scales, c.rows * 4, &scales, nullptr));
    HOLO_TRY(check_disjoint({ro, ib}, c.rope_output.slot, {{x, ib}, {co, ib}, {si, ib}, {codes, n}, {scales, c.rows * 4}}));
    HOLO_TRY(check_disjoint({codes, n}, c.codes.slot, {{x, ib}, {co, ib}, {si, ib}, {scales, c.rows * 4}}));
    HOLO_TRY(check_disjoint({scales, c.rows * 4}, c.scales.slot, {{x, ib}, {co, ib}, {si, ib}}));
    if (((uintptr_t)scales & 3u) != 0) return holo_fail_slot(c.scales.slot, "scales must be 4-byte aligned");
    return holo_launch_rope_quantize(ctx, x, co, si, ro, (int8_t*)codes, (float*)scales, c.rows, c.row_len, c.dtype);
}

// Geometry rules shared by both attention forms (cpu/float_kernels.rs:4192-4266).
int32_t attn_geometry(uint32_t b, uint32_t h, uint32_t kv, uint32_t m, uint32_t nnew, uint32_t d, uint32_t scale_bits,
                      uint32_t* hkv, float* scale_div, bool* empty) {
    *empty = (b == 0 || h == 0 || d == 0);
    if (*empty) return HOLO_OK;
    if (m == 0 || m != nnew)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP,
                         "unsupported op: decode_attention_valid: q_rows must equal new_len and be at least 1 "
                         "(the causal law pairs query row i with chunk key row i)");
    *hkv = kv == 0 ? h : kv;
    if (*hkv == 0 || h % *hkv != 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode_attention_valid: heads must be a multiple of kv_heads (grouped-query)");
    float dflt = sqrtf((float)d);
    if (dflt < 1.0f) dflt = 1.0f;
    *scale_div = dflt;
    if (scale_bits != 0) {
        float sm;
        memcpy(&sm, &scale_bits, 4);
        if (sm > 0.0f) *scale_div = 1.0f / sm;
    }
    return HOLO_OK;
}

// attention_float (cpu/float_kernels.rs:2244-2395): the prefill form. It is the decode row (:2420-2477) with an
// empty cache, the whole sequence as the chunk, and the causal law either on or off.
int32_t do_attention_legacy(holo_b200_ctx* ctx, const HoloAttentionCall& c, holo_b200_workspace* ws) {
    if (c.batch == 0 || c.heads == 0 || c.seq == 0 || c.head_dim == 0) return HOLO_OK;
    HoloAttnArgs a = {};
    a.hkv = c.kv_heads == 0 ? c.heads : c.kv_heads;
    if (c.heads % a.hkv != 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: attention: heads must be a multiple of kv_heads (grouped-query)");
    if (c.dtype == HOLO_DTYPE_F64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: f64 is not a supported compute dtype (hologram computes in f16/bf16/f32)");
    if (!holo_is_compute_float(c.dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: attention: only f32/f16/bf16 are supported compute dtypes");
    float dflt = sqrtf((float)c.head_dim);
    if (dflt < 1.0f) dflt = 1.0f;
    a.scale_div = dflt;
    if (c.scale_bits != 0) {
        float sm;
        memcpy(&sm, &c.scale_bits, 4);
        if (sm > 0.0f) a.scale_div = 1.0f / sm;
    }
    const size_t es = holo_dtype_size(c.dtype);
    const uint64_t qt = (uint64_t)c.batch * c.heads * c.seq * c.head_dim * es;
    const uint64_t kt = (uint64_t)c.batch * a.hkv * c.seq * c.head_dim * es;
    uint8_t *q, *k, *v, *out;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.q, qt, &q, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k, kt, &k, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v, kt, &v, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, qt, &out, nullptr));
    HOLO_TRY(check_disjoint({out, qt}, c.output.slot, {{q, qt}, {k, kt}, {v, kt}}));
    a.q = q; a.k_new = k; a.v_new = v; a.out = out;
    a.b = c.batch; a.h = c.heads; a.m = c.seq; a.past = 0; a.nnew = c.seq; a.d = c.head_dim;
    a.dtype = c.dtype;
    a.all_new = c.causal == 0;
    return holo_launch_decode_attention(ctx, a);
}

// decode_attention_valid_float (cpu/float_kernels.rs:4192-4307)
int32_t do_attention(holo_b200_ctx* ctx, const HoloDecodeAttentionValidCall& c, holo_b200_workspace* ws) {
    HoloAttnArgs a = {};
    bool empty;
    HOLO_TRY(attn_geometry(c.batch, c.heads, c.kv_heads, c.q_rows, c.new_len, c.head_dim, c.scale_bits, &a.hkv, &a.scale_div, &empty));
    if (empty) return HOLO_OK;
    if (c.dtype == HOLO_DTYPE_F64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: f64 is not a supported compute dtype (hologram computes in f16/bf16/f32)");
    if (!holo_is_compute_float(c.dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode_attention_valid: only f32/f16/bf16 are supported compute dtypes");
    size_t es = holo_dtype_size(c.dtype);
    uint64_t qt = (uint64_t)c.batch * c.heads * c.q_rows * c.head_dim * es;
    uint64_t pt = (uint64_t)c.batch * a.hkv * c.past_len * c.head_dim * es;
    uint64_t nt = (uint64_t)c.batch * a.hkv * c.new_len * c.head_dim * es;
    uint8_t *q, *kp, *vp, *kn, *vn, *vl, *out;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.q, qt, &q, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k_past, pt, &kp, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v_past, pt, &vp, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k_new, nt, &kn, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v_new, nt, &vn, nullptr));
    HOLO_TRY(holo_resolve(ws, c.valid_len, 4, &vl, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, qt, &out, nullptr));
    HOLO_TRY(check_disjoint({out, qt}, c.output.slot, {{q, qt}, {kp, pt}, {vp, pt}, {kn, nt}, {vn, nt}, {vl, 4}}));
    if (((uintptr_t)vl & 3u) != 0) return holo_fail_slot(c.valid_len.slot, "valid_len operand must be 4-byte aligned on the device");
    a.q = q; a.k_past = kp; a.v_past = vp; a.k_new = kn; a.v_new = vn;
    a.valid_len = (const uint32_t*)vl; a.out = out;
    a.b = c.batch; a.h = c.heads; a.m = c.q_rows; a.past = c.past_len; a.nnew = c.new_len; a.d = c.head_dim;
    a.dtype = c.dtype; a.quantized = false;
    return holo_launch_decode_attention(ctx, a);
}

// decode_attention_float, the additive-mask form (cpu/float_kernels.rs:2482-2600)
int32_t do_attention_mask(holo_b200_ctx* ctx, const HoloDecodeAttentionCall& c, holo_b200_workspace* ws) {
    if (c.batch == 0 || c.heads == 0 || c.q_rows == 0 || c.head_dim == 0) return HOLO_OK;
    const uint64_t l = (uint64_t)c.past_len + c.new_len;
    if (l == 0) return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode_attention: past_len + new_len must be at least 1");
    HoloAttnArgs a = {};
    a.hkv = c.kv_heads == 0 ? c.heads : c.kv_heads;
    if (a.hkv == 0 || c.heads % a.hkv != 0)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode_attention: heads must be a multiple of kv_heads (grouped-query)");
    if (c.dtype == HOLO_DTYPE_F64)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: f64 is not a supported compute dtype (hologram computes in f16/bf16/f32)");
    if (!holo_is_compute_float(c.dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode_attention: only f32/f16/bf16 are supported compute dtypes");
    a.scale_div = sqrtf((float)c.head_dim);
    if (a.scale_div < 1.0f) a.scale_div = 1.0f;
    if (c.scale_bits != 0) {
        float sm;
        memcpy(&sm, &c.scale_bits, 4);
        if (sm > 0.0f) a.scale_div = 1.0f / sm;
    }
    size_t es = holo_dtype_size(c.dtype);
    uint64_t qt = (uint64_t)c.batch * c.heads * c.q_rows * c.head_dim * es;
    uint64_t pt = (uint64_t)c.batch * a.hkv * c.past_len * c.head_dim * es;
    uint64_t nt = (uint64_t)c.batch * a.hkv * c.new_len * c.head_dim * es;
    uint64_t mt = (uint64_t)c.q_rows * l * 4;   // the mask is always f32
    uint8_t *q, *kp, *vp, *kn, *vn, *mk, *out;
    HOLO_TRY(holo_resolve(ws, c.output, 0, &out, nullptr));
    HOLO_TRY(holo_resolve(ws, c.q, qt, &q, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k_past, pt, &kp, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v_past, pt, &vp, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k_new, nt, &kn, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v_new, nt, &vn, nullptr));
    HOLO_TRY(holo_resolve(ws, c.mask, mt, &mk, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, qt, &out, nullptr));
    HOLO_TRY(check_disjoint({out, qt}, c.output.slot, {{q, qt}, {kp, pt}, {vp, pt}, {kn, nt}, {vn, nt}, {mk, mt}}));
    if (((uintptr_t)mk & 3u) != 0) return holo_fail_slot(c.mask.slot, "mask operand must be 4-byte aligned on the device");
    a.q = q; a.k_past = kp; a.v_past = vp; a.k_new = kn; a.v_new = vn;
    a.mask = (const float*)mk; a.out = out;
    a.b = c.batch; a.h = c.heads; a.m = c.q_rows; a.past = c.past_len; a.nnew = c.new_len; a.d = c.head_dim;
    a.dtype = c.dtype; a.quantized = false;
    return holo_launch_decode_attention(ctx, a);
}

int32_t do_attention_q8(holo_b200_ctx* ctx, const HoloDecodeAttentionValidQ8Call& c, holo_b200_workspace* ws) {
    HoloAttnArgs a = {};
    bool empty;
    HOLO_TRY(attn_geometry(c.batch, c.heads, c.kv_heads, c.q_rows, c.new_len, c.head_dim, c.scale_bits, &a.hkv, &a.scale_div, &empty));
    if (empty) return HOLO_OK;
    if (!holo_is_compute_float(c.dtype))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: decode_attention_valid_q8: q/output dtype must be f32, f16 or bf16");
    size_t es = holo_dtype_size(c.dtype);
    uint64_t qt = (uint64_t)c.batch * c.heads * c.q_rows * c.head_dim * es;
    uint64_t prow = (uint64_t)c.batch * a.hkv * c.past_len, nrow = (uint64_t)c.batch * a.hkv * c.new_len;
    uint64_t pt = prow * c.head_dim, nt = nrow * c.head_dim;
    uint8_t *q, *kp, *kps, *vp, *vps, *kn, *kns, *vn, *vns, *vl, *out;
    HOLO_TRY(holo_resolve(ws, c.q, qt, &q, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k_past, pt, &kp, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k_past_scales, prow * 4, &kps, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v_past, pt, &vp, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v_past_scales, prow * 4, &vps, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k_new, nt, &kn, nullptr));
    HOLO_TRY(holo_resolve(ws, c.k_new_scales, nrow * 4, &kns, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v_new, nt, &vn, nullptr));
    HOLO_TRY(holo_resolve(ws, c.v_new_scales, nrow * 4, &vns, nullptr));
    HOLO_TRY(holo_resolve(ws, c.valid_len, 4, &vl, nullptr));
    HOLO_TRY(holo_resolve(ws, c.output, qt, &out, nullptr));
    HOLO_TRY(check_disjoint({out, qt}, c.output.slot,
                            {{q, qt}, {kp, pt}, {vp, pt}, {kn, nt}, {vn, nt}, {kps, prow * 4}, {vps, prow * 4}, {kns, nrow * 4}, {vns, nrow * 4}, {vl, 4}}));
    if ((((uintptr_t)vl | (uintptr_t)kps | (uintptr_t)vps | (uintptr_t)kns | (uintptr_t)vns) & 3u) != 0)
        return holo_fail_slot(c.valid_len.slot, "valid_len and scale operands must be 4-byte aligned on the device");
    a.q = q; a.k_past = kp; a.v_past = vp; a.k_new = kn; a.v_new = vn;
    a.k_past_s = (const float*)kps; a.v_past_s = (const float*)vps; a.k_new_s = (const float*)kns; a.v_new_s = (const float*)vns;
    a.valid_len = (const uint32_t*)vl; a.out = out;
    a.b = c.batch; a.h = c.heads; a.m = c.q_rows; a.past = c.past_len; a.nnew = c.new_len; a.d = c.head_dim;
    a.dtype = c.dtype; a.quantized = true;
    return holo_launch_decode_attention(ctx, a);
}

int32_t do_all_reduce(holo_b200_ctx* ctx, const HoloAllReduceCall& c, holo_b200_workspace* ws) {
    size_t es = holo_dtype_size(c.dtype);
    if (c.dtype != HOLO_DTYPE_F32 && c.dtype != HOLO_DTYPE_BF16 && c.dtype != HOLO_DTYPE_F16)
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: all_reduce dtype %u", c.dtype);
    uint8_t* buf;
    HOLO_TRY(holo_resolve(ws, c.buffer, c.element_count * es, &buf, nullptr));
    return holo_all_reduce(ctx, buf, c.element_count, c.dtype);
}

}  // namespace

int32_t holo_dispatch_internal(holo_b200_ctx* ctx, const HoloKernelCall* call, holo_b200_workspace* ws) {
    int act = lut_act_of_kind(call->kind);
    if (act >= 0) return do_unary_lut(ctx, call->u.unary, act, ws);
    switch (call->kind) {
        case HOLO_K_ADD: return do_binary(ctx, call->u.binary, 0, ws);
        case HOLO_K_MUL: return do_binary(ctx, call->u.binary, 1, ws);
        case HOLO_K_MATMUL: return do_matmul(ctx, call->u.matmul, 0, nullptr, ws);
        case HOLO_K_MATMUL_ACTIVATION: return do_matmul(ctx, call->u.matmul_activation.mm, call->u.matmul_activation.act, nullptr, ws);
        case HOLO_K_MATMUL_ADD: return do_matmul(ctx, call->u.matmul_add.mm, 0, &call->u.matmul_add.residual, ws);
        case HOLO_K_MATMUL_ADD_ACTIVATION: return do_matmul_add_activation(ctx, call->u.matmul_add_activation, ws);
        case HOLO_K_MATMUL_DEQUANT_PLAIN: case HOLO_K_MATMUL_DEQUANT: case HOLO_K_MATMUL_DEQUANT_CODEBOOK:
            return do_matmul_dequant(ctx, call->u.matmul_dequant, ws);
        case HOLO_K_LAYER_NORM: return do_norm(ctx, call->u.norm, false, true, ws);
        case HOLO_K_RMS_NORM: return do_norm(ctx, call->u.norm, false, false, ws);
        case HOLO_K_ADD_RMS_NORM: return do_norm(ctx, call->u.norm, true, false, ws);
        case HOLO_K_SOFTMAX: return do_softmax(ctx, call->u.softmax, ws);
        case HOLO_K_ROTARY: return do_rope(ctx, call->u.rope, ws);
        case HOLO_K_GATHER: return do_gather(ctx, call->u.gather, ws);
        case HOLO_K_CAST: return do_cast(ctx, call->u.cast, ws);
        case HOLO_K_RESHAPE: case HOLO_K_SLICE: return do_reshape(ctx, call->u.layout, ws);
        case HOLO_K_CONCAT: return do_concat(ctx, call->u.binary, ws);
        case HOLO_K_TRANSPOSE: return do_transpose(ctx, call->u.transpose, ws);
        case HOLO_K_REDUCE_SUM: return do_reduce(ctx, call->u.reduce, 0, 0, ws);
        case HOLO_K_REDUCE_MEAN: return do_reduce(ctx, call->u.reduce, 0, 1, ws);
        case HOLO_K_REDUCE_PROD: return do_reduce(ctx, call->u.reduce, 1, 0, ws);
        case HOLO_K_REDUCE_MIN: return do_reduce(ctx, call->u.reduce, 2, 0, ws);
        case HOLO_K_REDUCE_MAX: return do_reduce(ctx, call->u.reduce, 3, 0, ws);
        case HOLO_K_EXPAND: {
            const HoloExpandCall& c = call->u.expand;
            return do_broadcast(ctx, "expand", c.input, nullptr, c.output, c.rank, c.in_dims, c.out_dims, -1, 1, c.dtype, ws);
        }
        case HOLO_K_BROADCAST_BINARY: {
            const HoloBroadcastBinaryCall& c = call->u.broadcast_binary;
            return do_broadcast(ctx, "broadcast_binary", c.small, &c.other, c.output, c.rank, c.in_dims, c.out_dims, c.op, c.small_is_lhs, c.dtype, ws);
        }
        case HOLO_K_DEQUANTIZE: return do_dequantize(ctx, call->u.dequantize, ws);
        case HOLO_K_KV_CACHE_WRITE: return do_kv_write(ctx, call->u.kv_cache_write, ws);
        case HOLO_K_WHERE: return do_where(ctx, call->u.where, ws);
        case HOLO_K_DEQUANT_ACTIVATION: return do_dequant_activation(ctx, call->u.dequant_activation, ws);
        case HOLO_K_ATTENTION: return do_attention_legacy(ctx, call->u.attention, ws);
        case HOLO_K_DECODE_ATTENTION: return do_attention_mask(ctx, call->u.decode_attention, ws);
        case HOLO_K_DECODE_ATTENTION_VALID: return do_attention(ctx, call->u.decode_attention_valid, ws);
        case HOLO_K_QUANTIZE_ROWS_I8: return do_quantize_rows(ctx, call->u.quantize_rows_i8, ws);
        case HOLO_K_DECODE_ATTENTION_VALID_Q8: return do_attention_q8(ctx, call->u.decode_attention_valid_q8, ws);
        case HOLO_K_ALL_REDUCE: return do_all_reduce(ctx, call->u.all_reduce, ws);
        case HOLO_K_ROPE_QUANTIZE_ROWS_I8: return do_rope_quantize(ctx, call->u.rope_quantize, ws);
        default:
            if (holo_is_exact_unary(call->kind) || holo_is_exact_binary(call->kind)) return do_elementwise(ctx, call, ws);
            return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: KernelCall variant %u is not served by the B200 backend (no CPU fallback)", call->kind);
    }
}

extern "C" int32_t holo_b200_dispatch(holo_b200_ctx* ctx, const HoloKernelCall* call, holo_b200_workspace* ws) {
    if (!ctx || !call || !ws) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: null argument");
    if (ws->ctx != ctx) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: workspace belongs to another context");
    HOLO_CUDA(cudaSetDevice(ctx->device));
    return holo_dispatch_internal(ctx, call, ws);
}

// ---- host-workspace form ---------------------------------------------------------------------
namespace {

}  // namespace

bool holo_collect_refs(HoloKernelCall* c, HoloRefList* l) {
    if (holo_is_exact_unary(c->kind)) {
        l->in(&c->u.unary.input);
        l->out(&c->u.unary.output, c->u.unary.element_count * holo_dtype_size(c->u.unary.dtype));
        return true;
    }
    if (holo_is_exact_binary(c->kind)) {
        l->in(&c->u.binary.a); l->in(&c->u.binary.b);
        l->out(&c->u.binary.output, c->u.binary.element_count * holo_dtype_size(c->u.binary.dtype));
        return true;
    }
    switch (c->kind) {
        case HOLO_K_SIGMOID: case HOLO_K_TANH: case HOLO_K_GELU: case HOLO_K_SILU: case HOLO_K_EXP: case HOLO_K_ERF:
            l->in(&c->u.unary.input);
            l->out(&c->u.unary.output, c->u.unary.element_count * holo_dtype_size(c->u.unary.dtype));
            return true;
        case HOLO_K_ADD: case HOLO_K_MUL:
            l->in(&c->u.binary.a); l->in(&c->u.binary.b);
            l->out(&c->u.binary.output, c->u.binary.element_count * holo_dtype_size(c->u.binary.dtype));
            return true;
        case HOLO_K_MATMUL: case HOLO_K_MATMUL_ACTIVATION: case HOLO_K_MATMUL_ADD: case HOLO_K_MATMUL_ADD_ACTIVATION: {
            // the four variants start with the same MatMulCall
            HoloMatMulCall& mm = c->u.matmul;
            l->in(&mm.a); l->in(&mm.b);
            if (c->kind == HOLO_K_MATMUL_ADD) l->in(&c->u.matmul_add.residual);
            if (c->kind == HOLO_K_MATMUL_ADD_ACTIVATION) l->in(&c->u.matmul_add_activation.residual);
            l->out(&mm.output, (uint64_t)mm.m * mm.n * holo_dtype_size(mm.dtype));
            return true;
        }
        case HOLO_K_ADD_RMS_NORM:
            l->in(&c->u.norm.residual);
            /* fall through */
        case HOLO_K_LAYER_NORM:
            l->in(&c->u.norm.beta);
            /* fall through */
        case HOLO_K_RMS_NORM:
            l->in(&c->u.norm.x); l->in(&c->u.norm.gamma);
            l->out(&c->u.norm.output, (uint64_t)c->u.norm.batch * c->u.norm.feature * holo_dtype_size(c->u.norm.dtype));
            return true;
        case HOLO_K_EXPAND: case HOLO_K_BROADCAST_BINARY: {
            const bool bin = c->kind == HOLO_K_BROADCAST_BINARY;
            const uint32_t* od = bin ? c->u.broadcast_binary.out_dims : c->u.expand.out_dims;
            const uint8_t rank = bin ? c->u.broadcast_binary.rank : c->u.expand.rank;
            uint64_t total = 1;
            for (uint32_t i = 0; i < rank && i < 8; ++i) total *= od[i];
            if (bin) {
                l->in(&c->u.broadcast_binary.small); l->in(&c->u.broadcast_binary.other);
                l->out(&c->u.broadcast_binary.output, total * holo_dtype_size(c->u.broadcast_binary.dtype));
            } else {
                l->in(&c->u.expand.input);
                l->out(&c->u.expand.output, total * holo_dtype_size(c->u.expand.dtype));
            }
            return true;
        }
        case HOLO_K_REDUCE_SUM: case HOLO_K_REDUCE_MEAN: case HOLO_K_REDUCE_PROD: case HOLO_K_REDUCE_MIN: case HOLO_K_REDUCE_MAX:
            l->in(&c->u.reduce.input);
            l->out(&c->u.reduce.output, reduce_out_count(c->u.reduce) * holo_dtype_size(c->u.reduce.dtype));
            return true;
        case HOLO_K_ATTENTION: {
            HoloAttentionCall& t = c->u.attention;
            l->in(&t.q); l->in(&t.k); l->in(&t.v);
            l->out(&t.output, (uint64_t)t.batch * t.heads * t.seq * t.head_dim * holo_dtype_size(t.dtype));
            return true;
        }
        case HOLO_K_WHERE:
            l->in(&c->u.where.cond); l->in(&c->u.where.a); l->in(&c->u.where.b);
            l->out(&c->u.where.output, c->u.where.element_count * holo_dtype_size(c->u.where.dtype));
            return true;
        case HOLO_K_DEQUANT_ACTIVATION:
            l->in(&c->u.dequant_activation.input);
            l->out(&c->u.dequant_activation.output, c->u.dequant_activation.element_count * 4);
            return true;
        case HOLO_K_SOFTMAX:
            l->in(&c->u.softmax.input);
            l->out(&c->u.softmax.output, (uint64_t)c->u.softmax.batch * c->u.softmax.feature * holo_dtype_size(c->u.softmax.dtype));
            return true;
        case HOLO_K_ROTARY:
            l->in(&c->u.rope.x); l->in(&c->u.rope.cos); l->in(&c->u.rope.sin);
            l->out(&c->u.rope.output, c->u.rope.element_count * holo_dtype_size(c->u.rope.dtype));
            return true;
        case HOLO_K_GATHER:
            l->in(&c->u.gather.data); l->in(&c->u.gather.indices);
            l->out(&c->u.gather.output, c->u.gather.outer * c->u.gather.num_indices * c->u.gather.inner * holo_dtype_size(c->u.gather.dtype));
            return true;
        case HOLO_K_CAST:
            l->in(&c->u.cast.input);
            l->out(&c->u.cast.output, c->u.cast.element_count * holo_dtype_size(c->u.cast.dst_dtype));
            return true;
        case HOLO_K_CONCAT: {
            auto& b = c->u.binary;
            l->in(&b.a); l->in(&b.b);
            // produced bytes = |a| + |b| when both extents are explicit (host staging needs them)
            l->out(&b.output, b.a.length && b.b.length ? b.a.length + b.b.length : b.output.length);
            return true;
        }
        case HOLO_K_TRANSPOSE: {
            auto& t = c->u.transpose;
            uint64_t total = holo_dtype_size(t.dtype);
            for (uint32_t i = 0; i < t.rank && i < 8; ++i) total *= t.dims[i];
            l->in(&t.input);
            l->out(&t.output, total);
            return true;
        }
        case HOLO_K_SLICE:
        case HOLO_K_RESHAPE:
            l->in(&c->u.layout.input);
            l->out(&c->u.layout.output, c->u.layout.element_count * holo_dtype_size(c->u.layout.dtype));
            return true;
        case HOLO_K_DEQUANTIZE:
            l->in(&c->u.dequantize.input); l->in(&c->u.dequantize.scales); l->in(&c->u.dequantize.zero_points);
            l->out(&c->u.dequantize.output, c->u.dequantize.element_count * holo_dtype_size(c->u.dequantize.dtype));
            return true;
        case HOLO_K_KV_CACHE_WRITE: {
            auto& k = c->u.kv_cache_write;
            l->in(&k.cache); l->in(&k.new_rows_buf); l->in(&k.pos);
            l->out(&k.output, (uint64_t)k.planes * k.bucket_rows * k.row_bytes);
            return true;
        }
        case HOLO_K_DECODE_ATTENTION: {
            auto& a = c->u.decode_attention;
            l->in(&a.q); l->in(&a.k_past); l->in(&a.v_past); l->in(&a.k_new); l->in(&a.v_new); l->in(&a.mask);
            l->out(&a.output, (uint64_t)a.batch * a.heads * a.q_rows * a.head_dim * holo_dtype_size(a.dtype));
            return true;
        }
        case HOLO_K_DECODE_ATTENTION_VALID: {
            auto& a = c->u.decode_attention_valid;
            l->in(&a.q); l->in(&a.k_past); l->in(&a.v_past); l->in(&a.k_new); l->in(&a.v_new); l->in(&a.valid_len);
            l->out(&a.output, (uint64_t)a.batch * a.heads * a.q_rows * a.head_dim * holo_dtype_size(a.dtype));
            return true;
        }
        case HOLO_K_QUANTIZE_ROWS_I8: {
            auto& q = c->u.quantize_rows_i8;
            l->in(&q.input);
            l->out(&q.codes, q.rows * q.row_len);
            l->out(&q.scales, q.rows * 4);
            return true;
        }
        case HOLO_K_DECODE_ATTENTION_VALID_Q8: {
            auto& a = c->u.decode_attention_valid_q8;
            l->in(&a.q); l->in(&a.k_past); l->in(&a.k_past_scales); l->in(&a.v_past); l->in(&a.v_past_scales);
            l->in(&a.k_new); l->in(&a.k_new_scales); l->in(&a.v_new); l->in(&a.v_new_scales); l->in(&a.valid_len);
            l->out(&a.output, (uint64_t)a.batch * a.heads * a.q_rows * a.head_dim * holo_dtype_size(a.dtype));
            return true;
        }
        case HOLO_K_ROPE_QUANTIZE_ROWS_I8: {
            auto& q = c->u.rope_quantize;
            l->in(&q.x); l->in(&q.cos); l->in(&q.sin);
            l->out(&q.rope_output, q.rows * q.row_len * holo_dtype_size(q.dtype));
            l->out(&q.codes, q.rows * q.row_len);
            l->out(&q.scales, q.rows * 4);
            return true;
        }
        case HOLO_K_MATMUL_DEQUANT_PLAIN: case HOLO_K_MATMUL_DEQUANT: case HOLO_K_MATMUL_DEQUANT_CODEBOOK: {
            auto& q = c->u.matmul_dequant;
            l->in(&q.a); l->in(&q.bq); l->in(&q.scales); l->in(&q.zero_points); l->in(&q.residual);
            if (c->kind == HOLO_K_MATMUL_DEQUANT_CODEBOOK) l->in(&q.codebook);
            l->out(&q.output, (uint64_t)q.m * q.n * holo_dtype_size(q.dtype));
            return true;
        }
        case HOLO_K_ALL_REDUCE:
            l->out(&c->u.all_reduce.buffer, c->u.all_reduce.element_count * holo_dtype_size(c->u.all_reduce.dtype));
            return true;
        default: return false;
    }
}



extern "C" int32_t holo_b200_dispatch_host(holo_b200_ctx* ctx, const HoloKernelCall* call, HoloHostSlot* host_slots, uint32_t n_slots) {
    if (!ctx || !call || !host_slots) return holo_fail(HOLO_ERR_DISPATCH, "dispatch failed: null argument");
    HOLO_CUDA(cudaSetDevice(ctx->device));
    HoloKernelCall local = *call;
    HoloRefList refs;
    if (!holo_collect_refs(&local, &refs))
        return holo_fail(HOLO_ERR_UNSUPPORTED_OP, "unsupported op: KernelCall variant %u has no host-workspace form", call->kind);
    // Each referenced host range gets a 256-byte aligned range of one device arena; the call
    // is rewritten to index a temporary device workspace with one slot per operand. Inputs
    // are uploaded whole; written operands are not uploaded and only the bytes the kernel
    // produces are copied back.
    uint64_t total = 0;
    uint64_t off[12], len[12];
    uint32_t orig_slot[12];
    uint8_t* host_ptr[12];
    for (int i = 0; i < refs.n; ++i) {
        HoloBufferRef r = *refs.refs[i];
        off[i] = len[i] = 0;
        orig_slot[i] = r.slot;
        host_ptr[i] = nullptr;
        if (r.slot == HOLO_NO_SLOT) continue;
        if (r.slot >= n_slots || !host_slots[r.slot].ptr) return holo_fail_slot(r.slot, "no such host slot");
        uint64_t sb = host_slots[r.slot].bytes;
        if (r.offset > sb) return holo_fail_slot(r.slot, "offset beyond slot");
        uint64_t ext = r.length ? r.length : sb - r.offset;
        if (ext > sb - r.offset) return holo_fail_slot(r.slot, "range beyond slot");
        if (refs.written[i] && refs.out_bytes[i] > ext) return holo_fail_slot(r.slot, "buffer shorter than the call's geometry requires");
        host_ptr[i] = (uint8_t*)host_slots[r.slot].ptr + r.offset;
        off[i] = total;
        len[i] = ext;
        total += (ext + 255) & ~255ull;
    }
    // split_borrow rule on the host ranges: a written range may not overlap any other operand
    for (int i = 0; i < refs.n; ++i) {
        if (!refs.written[i] || !host_ptr[i]) continue;
        for (int j = 0; j < refs.n; ++j) {
            if (j == i || !host_ptr[j] || len[j] == 0 || refs.out_bytes[i] == 0) continue;
            uint64_t lj = refs.written[j] ? refs.out_bytes[j] : len[j];
            if (host_ptr[j] < host_ptr[i] + refs.out_bytes[i] && host_ptr[i] < host_ptr[j] + lj)
                return holo_fail_slot(orig_slot[i], "output overlaps another operand");
        }
    }
    if (total > ctx->stage_bytes) {
        HOLO_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->stage) cudaFree(ctx->stage);
        ctx->stage = nullptr;
        ctx->stage_bytes = 0;
        HOLO_CUDA(cudaMalloc(&ctx->stage, total));
        ctx->stage_bytes = total;
    }
    holo_b200_workspace tmp;
    tmp.ctx = ctx;
    tmp.slots.resize(refs.n);
    for (int i = 0; i < refs.n; ++i) {
        HoloBufferRef& r = *refs.refs[i];
        if (r.slot == HOLO_NO_SLOT) continue;
        tmp.slots[i].ptr = (uint8_t*)ctx->stage + off[i];
        tmp.slots[i].bytes = len[i];
        if (!refs.written[i] && len[i])
            HOLO_CUDA(cudaMemcpyAsync(tmp.slots[i].ptr, host_ptr[i], len[i], cudaMemcpyHostToDevice, ctx->stream));
        r.slot = (uint32_t)i;
        r.offset = 0;
        r.length = len[i];
    }
    int32_t rc = holo_dispatch_internal(ctx, &local, &tmp);
    if (rc == HOLO_OK) {
        for (int i = 0; i < refs.n; ++i)
            if (refs.written[i] && host_ptr[i] && refs.out_bytes[i])
                HOLO_CUDA(cudaMemcpyAsync(host_ptr[i], tmp.slots[i].ptr, refs.out_bytes[i], cudaMemcpyDeviceToHost, ctx->stream));
        rc = check_dev_status(ctx);
    } else {
        cudaStreamSynchronize(ctx->stream);
        // report slot errors in the caller's slot numbering
        if (rc == HOLO_ERR_SLOT_OUT_OF_RANGE && g_err_slot < (uint32_t)refs.n) {
            uint32_t o = orig_slot[g_err_slot];
            char msg[400];
            snprintf(msg, sizeof msg, "%s", g_err);
            const char* paren = strchr(msg, '(');
            holo_fail_slot(o, paren ? "operand shorter than the call's geometry requires, or overlapping" : "slot error");
        }
    }
    return rc;
}
