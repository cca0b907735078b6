// Device-side numerics that must agree bit-for-bit with the reference CPU backend.
// Every float op that the reference performs as a separate IEEE operation is written with a
// round-to-nearest intrinsic (__fmul_rn / __fadd_rn / __fsub_rn / __fdiv_rn) so that nvcc
// never contracts a multiply-add into an FMA.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hologram_b200.h"

namespace holo {

__device__ __forceinline__ float bits_to_f32(uint32_t b) { return __uint_as_float(b); }
__device__ __forceinline__ uint32_t f32_to_bits(float f) { return __float_as_uint(f); }

// crates/hologram-compute/src/cpu/dtype.rs:69-79
__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16_trunc(float v) { return (uint16_t)(__float_as_uint(v) >> 16); }

// cpu/dtype.rs:94-118 (subnormals normalised, NaN payload shifted up)
__device__ __forceinline__ float f16_to_f32(uint16_t h) {
    uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1fu, mant = h & 0x3ffu, out;
    if (exp == 0) {
        if (mant == 0) {
            out = sign << 31;
        } else {
            int lz = __clz((int)mant) - 21;  // shifts needed to bring bit 10 up
            uint32_t m = mant << lz;
            int e = 1 - lz;
            out = (sign << 31) | ((uint32_t)(127 - 15 + e) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (exp == 0x1f) {
        out = (sign << 31) | (0xffu << 23) | (mant << 13);
    } else {
        out = (sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    return __uint_as_float(out);
}

// cpu/dtype.rs:121-153: add-half-then-shift rounding, one quiet NaN pattern, flush below 2^-25.
__device__ __forceinline__ uint16_t f32_to_f16_ref(float v) {
    uint32_t bits = __float_as_uint(v);
    uint32_t sign = (bits >> 31) & 1u;
    int exp = (int)((bits >> 23) & 0xffu);
    uint32_t mant = bits & 0x7fffffu;
    if (exp == 0xff) return (uint16_t)((sign << 15) | (0x1fu << 10) | (mant != 0 ? 0x200u : 0u));
    int new_exp = exp - 127 + 15;
    if (new_exp >= 0x1f) return (uint16_t)((sign << 15) | (0x1fu << 10));
    if (new_exp <= 0) {
        if (new_exp < -10) return (uint16_t)(sign << 15);
        uint32_t m = mant | 0x800000u;
        uint32_t shift = (uint32_t)(1 - new_exp) + 13u;
        uint32_t rounded = (m + (1u << (shift - 1))) >> shift;
        return (uint16_t)((sign << 15) | rounded);
    }
    uint32_t rounded_mant = (mant + 0x1000u) >> 13;
    if (rounded_mant & 0x400u) {
        int bumped = new_exp + 1;
        if (bumped >= 0x1f) return (uint16_t)((sign << 15) | (0x1fu << 10));
        return (uint16_t)((sign << 15) | ((uint32_t)bumped << 10));
    }
    return (uint16_t)((sign << 15) | ((uint32_t)new_exp << 10) | (rounded_mant & 0x3ffu));
}

__device__ __forceinline__ float widen16(uint16_t h, int dtype) {
    return dtype == HOLO_DTYPE_BF16 ? bf16_to_f32(h) : f16_to_f32(h);
}
__device__ __forceinline__ uint16_t narrow16(float v, int dtype) {
    return dtype == HOLO_DTYPE_BF16 ? f32_to_bf16_trunc(v) : f32_to_f16_ref(v);
}
// read_float / write_float (cpu/dtype.rs:156-181)
__device__ __forceinline__ float load_float(const void* p, uint64_t i, int dtype) {
    if (dtype == HOLO_DTYPE_F32) return ((const float*)p)[i];
    return widen16(((const uint16_t*)p)[i], dtype);
}
__device__ __forceinline__ void store_float(void* p, uint64_t i, float v, int dtype) {
    if (dtype == HOLO_DTYPE_F32) ((float*)p)[i] = v;
    else ((uint16_t*)p)[i] = narrow16(v, dtype);
}

// exp_f32_det, cpu/simd.rs:4191-4239. `(t ± 0.5) as i32` is a saturating truncation with
// NaN -> 0, which is exactly cvt.rzi.s32.f32.
__device__ __forceinline__ float exp_det(float x) {
    if (x != x || x < -87.33654f) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    float t = __fmul_rn(x, 1.44269504088896340736f);
    int k = t >= 0.0f ? __float2int_rz(__fadd_rn(t, 0.5f)) : __float2int_rz(__fsub_rn(t, 0.5f));
    float kf = __int2float_rn(k);
    float r = __fsub_rn(__fsub_rn(x, __fmul_rn(kf, __uint_as_float(0x3F318000u))), __fmul_rn(kf, -2.1219444e-4f));
    float p = 1.0f / 720.0f;
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 120.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 24.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f / 6.0f);
    p = __fadd_rn(__fmul_rn(p, r), 0.5f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    uint32_t sb = ((uint32_t)(k + 127)) << 23;
    if (sb > 0x7f000000u) sb = 0x7f000000u;
    return __fmul_rn(p, __uint_as_float(sb));
}

// cpu/float_kernels.rs:3548-3566
__device__ __forceinline__ float sigmoid_ref(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_det(-x))); }
__device__ __forceinline__ float tanh_ref(float x) {
    float e = exp_det(__fmul_rn(2.0f, x));
    return __fdiv_rn(__fsub_rn(e, 1.0f), __fadd_rn(e, 1.0f));
}
__device__ __forceinline__ float gelu_ref(float x) {
    // 0.5 * x * (1.0 + tanh_f(0.7978846 * (x + 0.044715 * x * x * x))), left to right
    float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, x), x), x);
    float inner = __fmul_rn(0.7978846f, __fadd_rn(x, cube));
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanh_ref(inner)));
}
__device__ __forceinline__ float silu_ref(float x) { return __fmul_rn(x, sigmoid_ref(x)); }
// Stand-ins for libm::expf / libm::erff (crate libm 0.2.16, cpu/float_kernels.rs:3498-3500,
// 3534-3536): the f32 rounding of the f64 function.
__device__ __forceinline__ float exp_standin(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float erf_standin(float x) { return (float)erf((double)x); }

// lut_act_ref, cpu/float_kernels.rs:3628-3638.
// NaN results follow the x86-64 SSE convention the reference's CPU tables are built under
// (CUDA arithmetic would return the canonical 0x7fffffff instead): an operation with a NaN
// operand returns that NaN quieted (payload and sign kept), an invalid operation such as
// 0 * inf returns the default NaN 0xFFC00000.
__device__ __forceinline__ float lut_act_ref(int act, float x) {
    float y;
    switch (act) {
        case HOLO_LUT_SIGMOID: y = sigmoid_ref(x); break;
        case HOLO_LUT_TANH: y = tanh_ref(x); break;
        case HOLO_LUT_GELU: y = gelu_ref(x); break;
        case HOLO_LUT_SILU: y = silu_ref(x); break;
        case HOLO_LUT_EXP: y = exp_standin(x); break;
        default: y = erf_standin(x); break;
    }
    if (y != y) y = (x != x) ? __uint_as_float(__float_as_uint(x) | 0x00400000u) : __uint_as_float(0xFFC00000u);
    return y;
}

// Elementwise float forms that are exact IEEE operations (cpu/float_kernels.rs:3446-3500 unary, :3660-3733
// binary), keyed by the call's wire discriminant. NaN results follow the x86-64 SSE convention the CPU
// backend runs under (see lut_act_ref): an arithmetic result that is NaN is the first NaN operand
// quieted, or the default NaN 0xFFC00000 for an invalid operation.
__device__ __forceinline__ float quiet_nan(float x) { return __uint_as_float(__float_as_uint(x) | 0x00400000u); }
__device__ __forceinline__ float nan_fix2(float y, float a, float b) {
    if (y == y) return y;
    return a != a ? quiet_nan(a) : b != b ? quiet_nan(b) : __uint_as_float(0xFFC00000u);
}
// f32::min / f32::max: the other operand when one is NaN; of two equal operands (+0 and -0) the first
__device__ __forceinline__ float min_ref(float a, float b) { return a != a ? b : (b < a ? b : a); }
__device__ __forceinline__ float max_ref(float a, float b) { return a != a ? b : (b > a ? b : a); }
// Neg and Abs are bit operations on the CPU (a NaN keeps its payload). Written as integer PTX so that the
// compiler cannot fold them into neg.f32 / abs.f32, which return the canonical NaN.
__device__ __forceinline__ float sign_bits(float x, uint32_t mask, bool clear) {
    uint32_t r;
    if (clear) asm volatile("and.b32 %0, %1, %2;" : "=r"(r) : "r"(__float_as_uint(x)), "r"(mask));
    else asm volatile("xor.b32 %0, %1, %2;" : "=r"(r) : "r"(__float_as_uint(x)), "r"(mask));
    return __uint_as_float(r);
}
__device__ __forceinline__ bool ew_is_unary(int tag) {
    return tag == 1 || tag == 11 || tag == 21 || tag == 22 || (tag >= 29 && tag <= 31) || (tag >= 33 && tag <= 35);
}
// Ceil / Floor / Round: the software libm the CPU backend links returns every |x| >= 2^23, a NaN included, unchanged.
__device__ __forceinline__ float ew_unary(int tag, float x) {
    switch (tag) {
        case 1: return sign_bits(x, 0x80000000u, false);                                        // Neg
        case 11: return max_ref(x, 0.0f);                                                       // Relu: x.max(0.0)
        case 21: return nan_fix2(__fsqrt_rn(x), x, x);                                          // Sqrt
        case 22: return nan_fix2(__fdiv_rn(1.0f, x), x, x);                                     // Reciprocal
        case 29: return x != x ? x : ceilf(x);
        case 30: return x != x ? x : floorf(x);
        case 31: return x != x ? x : roundf(x);   // half away from zero
        case 33: return x != x ? 1.0f : 0.0f;                                                   // IsNaN
        case 34: return x > 0.0f ? 1.0f : x < 0.0f ? -1.0f : 0.0f;                              // Sign
        default: return sign_bits(x, 0x7fffffffu, true);                                        // Abs
    }
}
__device__ __forceinline__ float ew_binary(int tag, float a, float b) {
    switch (tag) {
        case 6: return nan_fix2(__fsub_rn(a, b), a, b);
        case 36: return nan_fix2(__fdiv_rn(a, b), a, b);
        case 38: {   // floored modulo: a - floor(a / b) * b, every step rounded
            const float d = nan_fix2(__fdiv_rn(a, b), a, b);
            const float f = nan_fix2(floorf(d), d, d);
            const float m = nan_fix2(__fmul_rn(f, b), f, b);
            return nan_fix2(__fsub_rn(a, m), a, m);
        }
        case 39: return min_ref(a, b);
        case 40: return max_ref(a, b);
        case 41: return a == b ? 1.0f : 0.0f;
        case 42: return a < b ? 1.0f : 0.0f;
        case 43: return a <= b ? 1.0f : 0.0f;
        case 44: return a > b ? 1.0f : 0.0f;
        default: return a >= b ? 1.0f : 0.0f;
    }
}

}  // namespace holo
