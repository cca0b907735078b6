"""numpy front end to the CPU oracle (oracle/hologram_oracle.c).

TEST INFRASTRUCTURE ONLY: loaded by tests/, by __graft_entry__.smoke() and by bench.py's
CPU-baseline legs. The product package never imports this module.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

DTYPE_I8, DTYPE_I32, DTYPE_I64, DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 2, 4, 5, 6, 7, 8
_c = C.c_void_p


def _load(path):
    lib = C.CDLL(path)
    u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
    sig = {
        "holo_or_bf16_to_f32": (C.c_float, [C.c_uint16]),
        "holo_or_f32_to_bf16": (C.c_uint16, [C.c_float]),
        "holo_or_f16_to_f32": (C.c_float, [C.c_uint16]),
        "holo_or_f32_to_f16": (C.c_uint16, [C.c_float]),
        "holo_or_exp_det": (C.c_float, [C.c_float]),
        "holo_or_act": (C.c_float, [C.c_int, C.c_float]),
        "holo_or_build_table": (None, [C.c_int, C.c_int, u16p]),
        "holo_or_unary_lut": (C.c_int, [C.c_int, C.c_int, _c, _c, C.c_uint64]),
        "holo_or_unary_lut_mt": (C.c_int, [C.c_int, C.c_int, _c, _c, C.c_uint64]),
        "holo_or_quantize_row_i8": (C.c_float, [_c, _c, C.c_size_t]),
        "holo_or_quantize_rows_i8": (C.c_int, [_c, C.c_int, C.c_uint64, C.c_uint32, _c, _c]),
        "holo_or_matmul_i8_pc_omajor": (None, [_c, _c, _c, _c, C.c_size_t, C.c_size_t, C.c_size_t]),
        "holo_or_dequantize": (C.c_int, [_c, C.c_int, _c, _c, C.c_uint32, C.c_uint32, C.c_float, C.c_int32, _c,
                                          C.c_int, C.c_uint64]),
        "holo_or_cast_float": (C.c_int, [_c, C.c_int, _c, C.c_int, C.c_uint64]),
        "holo_or_matmul": (C.c_int, [_c, _c, _c, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]),
        "holo_or_matmul_activation": (C.c_int, [_c, _c, _c, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.c_int]),
        "holo_or_matmul_add": (C.c_int, [_c, _c, _c, _c, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]),
        "holo_or_matmul_add_activation": (C.c_int, [_c, _c, _c, _c, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.c_int]),
        "holo_or_matmul_dequant_kn": (C.c_int, [_c, _c, _c, _c, _c, _c, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int,
                                                C.c_float, C.c_int32, C.c_int]),
        "holo_or_binary": (C.c_int, [C.c_int, _c, _c, _c, C.c_uint64, C.c_int]),
        "holo_or_rms_norm": (C.c_int, [_c, _c, _c, C.c_uint32, C.c_uint32, C.c_uint64, C.c_int]),
        "holo_or_add_rms_norm": (C.c_int, [_c, _c, _c, _c, C.c_uint32, C.c_uint32, C.c_uint64, C.c_int]),
        "holo_or_matmul_e8cb_omajor": (None, [_c, _c, _c, _c, _c, C.c_size_t, C.c_size_t, C.c_size_t]),
        "holo_or_matmul_i4_pc_omajor": (None, [_c, _c, _c, _c, C.c_size_t, C.c_size_t, C.c_size_t]),
        "holo_or_dequant_activation": (C.c_int, [_c, _c, C.c_uint64, C.c_int, C.c_int, C.c_float, C.c_int32]),
        "holo_or_where": (C.c_int, [_c, _c, _c, _c, C.c_uint64, C.c_int]),
        "holo_or_elementwise": (C.c_int, [C.c_int, _c, _c, _c, C.c_uint64, C.c_int]),
        "holo_or_reduce": (C.c_int, [_c, _c, C.c_uint64, C.c_uint32, _c, C.c_uint32, C.c_int, C.c_int, C.c_int]),
        "holo_or_broadcast": (C.c_int, [_c, _c, _c, C.c_uint32, _c, _c, C.c_uint32, C.c_int, C.c_int, C.c_int]),
        "holo_or_layer_norm": (C.c_int, [_c, _c, _c, _c, C.c_uint32, C.c_uint32, C.c_uint64, C.c_int]),
        "holo_or_softmax": (C.c_int, [_c, _c, C.c_uint32, C.c_uint32, C.c_int]),
        "holo_or_transpose": (C.c_int, [_c, _c, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint8), C.c_uint32]),
        "holo_or_rope": (C.c_int, [_c, _c, _c, _c, C.c_uint32, C.c_uint64, C.c_int]),
        "holo_or_gather": (C.c_int, [_c, _c, C.c_int, _c, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int]),
        "holo_or_kv_cache_write": (C.c_int, [_c, _c, C.c_uint32, _c, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
        "holo_or_decode_attention_valid_f32": (C.c_int, [_c] * 5 + [C.c_uint32, _c] + [C.c_uint32] * 8),
        "holo_or_decode_attention_valid": (C.c_int, [_c] * 5 + [C.c_uint32, _c] + [C.c_uint32] * 8 + [C.c_int]),
        "holo_or_decode_attention_mask": (C.c_int, [_c] * 7 + [C.c_uint32] * 8 + [C.c_int]),
        "holo_or_decode_attention_valid_q8": (C.c_int, [_c, C.c_int] + [_c] * 8 + [C.c_uint32, _c] + [C.c_uint32] * 8),
        "holo_or_fnv1a64_f32": (C.c_uint64, [_c, C.c_size_t]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_PARITY, _FAST = _build.build()
lib = _load(_PARITY)
_fast = None


def fast_lib():
    """The -O3 build, for timed CPU-baseline legs only."""
    global _fast
    if _fast is None:
        _fast = _load(_FAST)
    return _fast


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _np_store(dtype):
    return np.float32 if dtype == DTYPE_F32 else np.uint16


def build_table(act, dtype):
    t = np.empty(65536, dtype=np.uint16)
    lib.holo_or_build_table(act, dtype, t)
    return t


def unary_lut(act, dtype, x_bits, which=None, mt=False):
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    out = np.empty_like(x)
    L = which or lib
    fn = L.holo_or_unary_lut_mt if mt else L.holo_or_unary_lut
    rc = fn(act, dtype, _p(x), _p(out), x.size)
    assert rc == 0, rc
    return out


def f32_to_bf16_trunc(x):
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_to_f32(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_rne(x):
    """Round-to-nearest-even narrowing, for input synthesis only (outputs truncate)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    r[nan] = 0x7FC0
    return r


def quantize_rows_i8(x, dtype, rows, d):
    x = np.ascontiguousarray(x)
    codes = np.zeros(rows * d, dtype=np.int8)
    scales = np.zeros(rows, dtype=np.float32)
    rc = lib.holo_or_quantize_rows_i8(_p(x), dtype, rows, d, _p(codes), _p(scales))
    assert rc == 0, rc
    return codes, scales


def matmul(a, b, m, k, n, dtype, act=0, residual=None, which=None):
    L = which or lib
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    out = np.zeros(m * n, dtype=_np_store(dtype))
    if residual is not None:
        r = np.ascontiguousarray(residual)
        rc = L.holo_or_matmul_add(_p(a), _p(b), _p(r), _p(out), m, k, n, dtype)
    elif act:
        rc = L.holo_or_matmul_activation(_p(a), _p(b), _p(out), m, k, n, dtype, act)
    else:
        rc = L.holo_or_matmul(_p(a), _p(b), _p(out), m, k, n, dtype)
    assert rc == 0, rc
    return out


def matmul_add_activation(a, b, residual, m, k, n, dtype, act):
    """matmul_add_activation_float (cpu/float_kernels.rs:899-938); act is a fused_activation id."""
    a, b, r = (np.ascontiguousarray(v) for v in (a, b, residual))
    out = np.zeros(m * n, dtype=_np_store(dtype))
    rc = lib.holo_or_matmul_add_activation(_p(a), _p(b), _p(r), _p(out), m, k, n, dtype, act)
    assert rc == 0, rc
    return out


def matmul_dequant_kn(a, bq, m, k, n, quant_dtype, scales=None, zero_points=None, channels=0, inner=1, scale=1.0, zero_point=0,
                      residual=None, act=None):
    """matmul_dequant_float over a [k, n] weight with f32 activations (cpu/float_kernels.rs:596-770); act is a LUT id."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bq = np.ascontiguousarray(bq).view(np.uint8)
    sc = None if scales is None else np.ascontiguousarray(scales, dtype=np.float32)
    zp = None if zero_points is None else np.ascontiguousarray(zero_points, dtype=np.int32)
    res = None if residual is None else np.ascontiguousarray(residual, dtype=np.float32)
    out = np.zeros(m * n, dtype=np.float32)
    rc = lib.holo_or_matmul_dequant_kn(_p(a), _p(bq), _p(sc), _p(zp), _p(res), _p(out), m, k, n, channels, inner, quant_dtype,
                                       float(np.float32(scale)), zero_point, -1 if act is None else act)
    assert rc == 0, rc
    return out


def binary(op, a, b, dtype):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    out = np.empty_like(a)
    assert lib.holo_or_binary(op, _p(a), _p(b), _p(out), a.size, dtype) == 0
    return out


def dequant_activation(codes, n, quant_dtype, act, scale, zero_point):
    codes = np.ascontiguousarray(codes).view(np.uint8)
    out = np.empty(n, dtype=np.float32)
    rc = lib.holo_or_dequant_activation(_p(codes), _p(out), n, quant_dtype, act, float(np.float32(scale)), zero_point)
    assert rc == 0, rc
    return out


def attention(q, k, v, b, h, kv, seq, d, causal, scale_bits, dtype):
    """attention_float (cpu/float_kernels.rs:2244-2395). Its per-row arithmetic (:2352-2388: dot / scale, -inf for the
    keys the causal law hides, max shift, deterministic exp, left-to-right sum, e / max(sum, 1e-30), context in key
    order) is the decode row (:2420-2477) with an empty cache, the sequence as the chunk and a 0 / -inf mask."""
    mask = np.zeros((seq, seq), dtype=np.float32)
    if causal:
        mask[np.triu_indices(seq, 1)] = -np.inf
    empty = np.zeros(0, dtype=np.asarray(q).dtype)
    return decode_attention_mask(q, empty, empty, k, v, mask, b, h, kv, seq, 0, seq, d, scale_bits, dtype)


def where(cond, a, b, dtype):
    cond, a, b = (np.ascontiguousarray(v) for v in (cond, a, b))
    out = np.empty_like(a)
    assert lib.holo_or_where(_p(cond.view(np.uint8)), _p(a), _p(b), _p(out), a.size, dtype) == 0
    return out


def elementwise(tag, a, b, dtype):
    """The exact unary (b None) and binary variants, by wire discriminant."""
    a = np.ascontiguousarray(a)
    b = None if b is None else np.ascontiguousarray(b)
    out = np.empty_like(a)
    rc = lib.holo_or_elementwise(tag, _p(a), _p(b), _p(out), a.size, dtype)
    assert rc == 0, rc
    return out


def rms_norm(x, gamma, batch, feature, eps_bits, dtype):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    g = None if gamma is None else np.ascontiguousarray(gamma)
    rc = lib.holo_or_rms_norm(_p(x), _p(g), _p(out), batch, feature, eps_bits, dtype)
    assert rc == 0, rc
    return out


def decode_attention_mask(q, kp, vp, kn, vn, mask, b, h, kv, m, past, new, d, scale_bits, dtype):
    """The additive-mask form (kernel_call.rs:632-655); operands flat, mask f32 [m, past + new]."""
    q, kp, vp, kn, vn = (np.ascontiguousarray(v) for v in (q, kp, vp, kn, vn))
    mask = np.ascontiguousarray(mask, dtype=np.float32)
    out = np.empty_like(q)
    rc = lib.holo_or_decode_attention_mask(_p(q), _p(kp), _p(vp), _p(kn), _p(vn), _p(mask), _p(out), b, h, kv, m, past, new, d,
                                           scale_bits, dtype)
    assert rc == 0, rc
    return out


def matmul_w8a8_omajor(a, bq, scales, m, k, n, residual=None, act=None, i4=False, codebook=None):
    """matmul_dequant_float, output-major W8A8 arm + epilogue (cpu/float_kernels.rs:534-596, 727-766):
    a f32 [m,k], bq i8 [n,k], scales f32 [n]; act is a LUT activation id applied by the scalar function."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bq = np.ascontiguousarray(bq, dtype=np.uint8 if (i4 or codebook is not None) else np.int8)   # i4: [n, k/2] packed nibbles (cpu/simd.rs:6164-6171)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    out = np.zeros(m * n, dtype=np.float32)
    if codebook is not None:     # E8 codebook tier: [n, k/8] indices into the model's 256 x 8 i8 codebook (cpu/simd.rs:6856-6861)
        cb = np.ascontiguousarray(codebook, dtype=np.int8)
        assert cb.size == 2048
        lib.holo_or_matmul_e8cb_omajor(_p(a), _p(bq), _p(cb), _p(scales), _p(out), m, k, n)
    else:
        (lib.holo_or_matmul_i4_pc_omajor if i4 else lib.holo_or_matmul_i8_pc_omajor)(_p(a), _p(bq), _p(scales), _p(out), m, k, n)
    if residual is not None:
        out = out + np.ascontiguousarray(residual, dtype=np.float32)
    if act is not None:
        out = np.array([lib.holo_or_act(act, float(v)) for v in out], dtype=np.float32)
    return out


def add_rms_norm(x, residual, gamma, batch, feature, eps_bits, dtype):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    r = None if residual is None else np.ascontiguousarray(residual)
    g = None if gamma is None else np.ascontiguousarray(gamma)
    rc = lib.holo_or_add_rms_norm(_p(x), _p(r), _p(g), _p(out), batch, feature, eps_bits, dtype)
    assert rc == 0, rc
    return out


def reduce(x, dims, axes_mask, kind, mean, dtype):
    """kind 0 sum, 1 prod, 2 min, 3 max; returns the keepdims-layout output cells."""
    x = np.ascontiguousarray(x)
    d = np.asarray(dims, dtype=np.uint32)
    cells = 1
    if len(dims) and axes_mask:
        for i, v in enumerate(dims):
            if not (axes_mask >> i) & 1:
                cells *= v
    out = np.zeros(cells, dtype=x.dtype)
    rc = lib.holo_or_reduce(_p(x), _p(out), x.size, len(dims), _p(d), axes_mask, kind, int(mean), dtype)
    assert rc == 0, rc
    return out


def broadcast(small, other, in_dims, out_dims, itemsize, op=-1, small_is_lhs=True, dtype=DTYPE_F32):
    """Expand (other None) or BroadcastBinary; returns the raw output bytes as uint8."""
    small = np.ascontiguousarray(small)
    other = None if other is None else np.ascontiguousarray(other)
    ind, outd = np.asarray(in_dims, dtype=np.uint32), np.asarray(out_dims, dtype=np.uint32)
    out = np.zeros(int(np.prod(outd, dtype=np.uint64)) * itemsize, dtype=np.uint8)
    rc = lib.holo_or_broadcast(_p(small), _p(other), _p(out), len(outd), _p(ind), _p(outd), itemsize, op, int(small_is_lhs), dtype)
    assert rc == 0, rc
    return out


def layer_norm(x, gamma, beta, batch, feature, eps_bits, dtype):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    g = None if gamma is None else np.ascontiguousarray(gamma)
    b = None if beta is None else np.ascontiguousarray(beta)
    rc = lib.holo_or_layer_norm(_p(x), _p(g), _p(b), _p(out), batch, feature, eps_bits, dtype)
    assert rc == 0, rc
    return out


def softmax(x, batch, feature, dtype):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    assert lib.holo_or_softmax(_p(x), _p(out), batch, feature, dtype) == 0
    return out


def transpose(x, dims, perm, itemsize):
    """x: flat array of prod(dims) elements of `itemsize` bytes; returns the permuted flat bytes."""
    import ctypes as C
    b = np.ascontiguousarray(x).view(np.uint8).reshape(-1)
    out = np.empty_like(b)
    d = (C.c_uint32 * 8)(*dims)
    pm = (C.c_uint8 * 8)(*perm)
    rc = lib.holo_or_transpose(_p(b), _p(out), len(dims), d, pm, itemsize)
    assert rc == 0, rc
    return out


def rope(x, cos, sin, head_dim, dtype):
    x, cos, sin = (np.ascontiguousarray(v) for v in (x, cos, sin))
    out = np.empty_like(x)
    rc = lib.holo_or_rope(_p(x), _p(cos), _p(sin), _p(out), head_dim, x.size, dtype)
    assert rc == 0, rc
    return out


def gather(data, idx, outer, axis_dim, inner, dtype):
    data = np.ascontiguousarray(data)
    idx = np.ascontiguousarray(idx)
    idt = DTYPE_I32 if idx.dtype == np.int32 else DTYPE_I64
    es = data.dtype.itemsize
    out = np.zeros(outer * idx.size * inner, dtype=data.dtype)
    rc = lib.holo_or_gather(_p(data), _p(idx), idt, _p(out), outer, axis_dim, inner, idx.size,
                            {1: 1, 2: DTYPE_BF16, 4: DTYPE_F32, 8: DTYPE_I64}[es])
    return rc, out


def kv_cache_write(cache, new, pos, planes, bucket, new_rows, row_bytes):
    cache = np.ascontiguousarray(cache).view(np.uint8)
    new = np.ascontiguousarray(new).view(np.uint8)
    out = np.empty_like(cache)
    rc = lib.holo_or_kv_cache_write(_p(cache), _p(new), pos, _p(out), planes, bucket, new_rows, row_bytes)
    return rc, out


def dequantize(codes, scales, zps, channels, inner, scale, zp, dtype, quant_dtype=DTYPE_I8):
    codes = np.ascontiguousarray(codes)
    out = np.zeros(codes.size, dtype=_np_store(dtype))
    s = None if scales is None else np.ascontiguousarray(scales, dtype=np.float32)
    z = None if zps is None else np.ascontiguousarray(zps, dtype=np.int32)
    rc = lib.holo_or_dequantize(_p(codes), quant_dtype, _p(s), _p(z), channels, inner, scale, zp, _p(out), dtype,
                                codes.size)
    assert rc == 0, rc
    return out


def cast_float(x, src, dst):
    x = np.ascontiguousarray(x)
    out = np.zeros(x.size, dtype=_np_store(dst))
    assert lib.holo_or_cast_float(_p(x), src, _p(out), dst, x.size) == 0
    return out


def decode_attention_valid(q, kp, vp, kn, vn, valid_len, b, h, kv, m, past, new, d, scale_bits, dtype, which=None):
    L = which or lib
    arrs = [np.ascontiguousarray(v) for v in (q, kp, vp, kn, vn)]
    out = np.zeros(b * h * m * d, dtype=_np_store(dtype))
    rc = L.holo_or_decode_attention_valid(*[_p(v) for v in arrs], valid_len, _p(out), b, h, kv, m, past, new, d,
                                          scale_bits, dtype)
    return rc, out


def decode_attention_valid_q8(q, dtype, kp, kps, vp, vps, kn, kns, vn, vns, valid_len, b, h, kv, m, past, new, d,
                              scale_bits, which=None):
    L = which or lib
    arrs = [np.ascontiguousarray(v) for v in (kp, kps, vp, vps, kn, kns, vn, vns)]
    q = np.ascontiguousarray(q)
    out = np.zeros(b * h * m * d, dtype=_np_store(dtype))
    rc = L.holo_or_decode_attention_valid_q8(_p(q), dtype, *[_p(v) for v in arrs], valid_len, _p(out), b, h, kv, m,
                                             past, new, d, scale_bits)
    return rc, out


def fnv1a64_f32(v):
    v = np.ascontiguousarray(v, dtype=np.float32)
    return int(lib.holo_or_fnv1a64_f32(_p(v), v.size))
