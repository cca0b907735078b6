"""The oracle against every known-answer value the reference's own tests hold for this path
(no GPU). File:line citations are into the reference tree."""
import math
import json
import os
import struct

import numpy as np
import pytest

from hologram_b200 import kernel_call as kc
from oracle import oracle as orc

L = orc.lib


def bits(f):
    return struct.unpack("<I", struct.pack("<f", f))[0]


def test_exp_det_edges_bit_exact():
    # crates/hologram-compute/src/cpu/simd.rs:7621-7624
    assert bits(L.holo_or_exp_det(0.0)) == bits(1.0)
    for x in (float("-inf"), float("nan"), -1000.0):
        assert bits(L.holo_or_exp_det(x)) == bits(0.0)
    assert bits(L.holo_or_exp_det(-0.0)) == bits(1.0)


def test_exp_det_accuracy():
    # simd.rs:7610-7620: relative error < 2e-6 against the true exponential on [-87, 88]
    v, worst = -87.0, 0.0
    while v <= 88.0:
        x = np.float32(v)
        e = float(L.holo_or_exp_det(float(x)))
        r = math.exp(float(x))
        worst = max(worst, abs(e - r) / r)
        v += 0.0173
    assert worst < 2e-6


def test_quantizer_pinned_by_the_w8a8_golden():
    # simd.rs:8236-8262: FNV-1a-64 over the W8A8 output-major GEMV output bits
    m, k, n = 3, 64, 24
    a = (np.array([float(i * 37 % 91) for i in range(m * k)], dtype=np.float32) - np.float32(45.0)) * np.float32(0.031)
    scales = np.float32(0.011) + np.arange(n, dtype=np.float32) * np.float32(0.0007)
    bq = np.array([(i * 31 % 255) - 127 for i in range(k * n)], dtype=np.int8)
    out = np.zeros(m * n, dtype=np.float32)
    L.holo_or_matmul_i8_pc_omajor(a.ctypes.data, bq.ctypes.data, scales.ctypes.data, out.ctypes.data, m, k, n)
    assert orc.fnv1a64_f32(out) == 0x787CCDC172029F9B


def test_bf16_narrow_truncates():
    # crates/hologram-compute/tests/dtype_codec.rs:19-32: bf16 write is bits >> 16, never rounds up
    x = struct.unpack("<f", struct.pack("<I", 0x3F80FFFF))[0]
    assert L.holo_or_f32_to_bf16(x) == 0x3F80
    for v in (1.0, -2.5, 3.140625, 1e-20, -7e30):
        h = L.holo_or_f32_to_bf16(v)
        assert h == bits(np.float32(v)) >> 16
        assert bits(L.holo_or_bf16_to_f32(h)) == (h << 16)


def test_f16_widen_matches_ieee_for_all_patterns():
    # cpu/dtype.rs:94-118 is an exact widening; numpy's float16 is the independent authority
    allbits = np.arange(65536, dtype=np.uint16)
    want = allbits.view(np.float16).astype(np.float32).view(np.uint32)
    got = np.array([bits(L.holo_or_f16_to_f32(int(b))) for b in allbits], dtype=np.uint32)
    nan = np.isnan(allbits.view(np.float16))
    assert np.array_equal(got[~nan], want[~nan])
    # NaN: payload shifted up by 13 bits (dtype.rs:112-114)
    assert np.array_equal(got[nan] & 0x7F800000, np.full(nan.sum(), 0x7F800000, dtype=np.uint32))


def test_f16_narrow_rule():
    # cpu/dtype.rs:121-153: add-half-then-shift (ties go up in magnitude), one NaN pattern,
    # overflow to inf, flush below 2^-25
    f = L.holo_or_f32_to_f16
    assert f(1.0) == 0x3C00 and f(-2.0) == 0xC000
    assert f(65520.0) == 0x7C00 and f(1e9) == 0x7C00 and f(-1e9) == 0xFC00
    assert f(float("nan")) & 0x7FFF == 0x7E00
    assert f(2.0 ** -26) == 0x0000 and f(-(2.0 ** -26)) == 0x8000
    # 1 + 2^-11 is a tie between 0x3C00 and 0x3C01: this codec rounds it up, RNE would not
    assert f(1.0 + 2.0 ** -11) == 0x3C01
    assert np.float32(1.0 + 2.0 ** -11).astype(np.float16).view(np.uint16) == 0x3C00
    # round trip of every finite f16 is the identity
    for b in list(range(0, 0x7C00, 37)) + list(range(0x8000, 0xFC00, 41)):
        assert f(L.holo_or_f16_to_f32(b)) == b


def test_lut_gelu_bf16_against_f64_reference():
    # crates/hologram-compute/tests/lut.rs:68-100
    n = 64
    x = np.array([i * 0.25 - 8.0 for i in range(n)], dtype=np.float32)
    xb = orc.f32_to_bf16_trunc(x)
    got = orc.bf16_to_f32(orc.unary_lut(kc.LUT_GELU, kc.DTYPE_BF16, xb))
    c = math.sqrt(2.0 / math.pi)
    for i in range(n):
        xv = float(orc.bf16_to_f32(xb[i:i + 1])[0])
        want = 0.5 * xv * (1.0 + math.tanh(c * (xv + 0.044715 * xv ** 3)))
        assert abs(float(got[i]) - want) <= 0.02 + 0.02 * abs(want)


def test_lut_sigmoid_bf16_against_f64_reference():
    # tests/lut.rs:103-132
    n = 48
    xb = orc.f32_to_bf16_trunc(np.array([i * 0.4 - 9.0 for i in range(n)], dtype=np.float32))
    got = orc.bf16_to_f32(orc.unary_lut(kc.LUT_SIGMOID, kc.DTYPE_BF16, xb))
    x = orc.bf16_to_f32(xb)
    for i in range(n):
        assert abs(float(got[i]) - 1.0 / (1.0 + math.exp(-float(x[i])))) <= 0.01


def test_table_special_values():
    # consequences of lut_act_ref + exp_f32_det (float_kernels.rs:3548-3566, simd.rs:4217-4239)
    bf = kc.DTYPE_BF16
    sig, tanh, gelu, silu = (orc.build_table(a, bf) for a in (kc.LUT_SIGMOID, kc.LUT_TANH, kc.LUT_GELU, kc.LUT_SILU))
    qnan = 0x7FC0
    assert sig[qnan] == 0x3F80            # 1 / (1 + exp_det(NaN) = 0) = 1.0
    assert tanh[qnan] == 0xBF80           # (0 - 1) / (0 + 1) = -1.0
    assert np.isnan(orc.bf16_to_f32(gelu[qnan:qnan + 1])[0])
    assert np.isnan(orc.bf16_to_f32(silu[qnan:qnan + 1])[0])
    assert tanh[0x7F80] == 0x3F80 and tanh[0x4120] == 0x3F80   # tanh(+inf) = tanh(10) = exactly 1.0
    assert sig[0x0000] == 0x3F00 and sig[0x8000] == 0x3F00     # sigmoid(±0) = 0.5
    exp_t = orc.build_table(kc.LUT_EXP, bf)
    assert exp_t[0x0000] == 0x3F80 and exp_t[0x8000] == 0x3F80 and exp_t[0xFF80] == 0x0000
    assert exp_t[0x7F80] == 0x7F80


def test_lut_is_the_table():
    for act in range(6):
        for dt in (kc.DTYPE_F16, kc.DTYPE_BF16):
            t = orc.build_table(act, dt)
            allbits = np.arange(65536, dtype=np.uint16)
            assert np.array_equal(orc.unary_lut(act, dt, allbits), t)


def test_quantize_row_edges():
    # all-zero row -> zero codes, scale 0.0 (simd.rs:4769-4771); clamp at ±127; half away from zero
    codes, scales = orc.quantize_rows_i8(np.zeros(8, dtype=np.float32), kc.DTYPE_F32, 1, 8)
    assert not codes.any() and scales[0] == 0.0
    x = np.array([127.0, -127.0, 0.5, -0.5, 1.5, -1.5, 0.49, 63.5], dtype=np.float32)
    codes, scales = orc.quantize_rows_i8(x, kc.DTYPE_F32, 1, 8)
    assert scales[0] == np.float32(127.0) / np.float32(127.0)
    assert codes.tolist() == [127, -127, 1, -1, 2, -2, 0, 64]


def _fixture(n, seed):
    # tests/decode_attention.rs:95-99 integer-formula corpus
    return np.array([(((i * 13 + seed * 7) % 41) - 20.0) * 0.043 for i in range(n)], dtype=np.float32)


def test_attention_witness_relations_on_oracle():
    # tests/decode_attention_valid.rs: garbage beyond valid_len is never read; valid_len >= past
    # means the whole bucket; zero visible past keys still sees the causal chunk.
    b, h, hkv, m, past, d = 1, 4, 2, 4, 12, 16
    q = _fixture(b * h * m * d, 1)
    kp, vp = _fixture(b * hkv * past * d, 2), _fixture(b * hkv * past * d, 3)
    kn, vn = _fixture(b * hkv * m * d, 4), _fixture(b * hkv * m * d, 5)
    f32 = kc.DTYPE_F32
    rc, full = orc.decode_attention_valid(q, kp, vp, kn, vn, past, b, h, hkv, m, past, m, d, 0, f32)
    assert rc == 0
    rc, over = orc.decode_attention_valid(q, kp, vp, kn, vn, 10 ** 6, b, h, hkv, m, past, m, d, 0, f32)
    assert np.array_equal(full.view(np.uint32), over.view(np.uint32))
    valid = 5
    kg, vg = kp.copy().reshape(b * hkv, past, d), vp.copy().reshape(b * hkv, past, d)
    kg[:, valid:, :] = np.nan
    vg[:, valid:, :] = np.nan
    rc, a = orc.decode_attention_valid(q, kg, vg, kn, vn, valid, b, h, hkv, m, past, m, d, 0, f32)
    tight_k = np.ascontiguousarray(kp.reshape(b * hkv, past, d)[:, :valid, :])
    tight_v = np.ascontiguousarray(vp.reshape(b * hkv, past, d)[:, :valid, :])
    rc, t = orc.decode_attention_valid(q, tight_k, tight_v, kn, vn, valid, b, h, hkv, m, valid, m, d, 0, f32)
    assert np.array_equal(a.view(np.uint32), t.view(np.uint32))   # padded == tight, bitwise
    assert not np.isnan(a).any()
    # q_rows != new_len is refused (float_kernels.rs:4205-4210)
    rc, _ = orc.decode_attention_valid(q, kp, vp, kn, vn, past, b, h, hkv, m, past, m - 1, d, 0, f32)
    assert rc == -3
    # heads not a multiple of kv_heads is refused (:4216-4220)
    rc, _ = orc.decode_attention_valid(q, kp, vp, kn, vn, past, b, h, 3, m, past, m, d, 0, f32)
    assert rc == -3


def test_attention_against_independent_f64_softmax():
    b, h, hkv, m, past, d = 2, 4, 2, 1, 9, 8
    rng = np.random.default_rng(5)
    q = rng.standard_normal(b * h * m * d).astype(np.float32)
    kp, vp = (rng.standard_normal(b * hkv * past * d).astype(np.float32) for _ in range(2))
    kn, vn = (rng.standard_normal(b * hkv * m * d).astype(np.float32) for _ in range(2))
    rc, got = orc.decode_attention_valid(q, kp, vp, kn, vn, 7, b, h, hkv, m, past, m, d, 0, kc.DTYPE_F32)
    assert rc == 0
    Q = q.reshape(b, h, d).astype(np.float64)
    K = np.concatenate([kp.reshape(b, hkv, past, d)[:, :, :7], kn.reshape(b, hkv, 1, d)], axis=2).astype(np.float64)
    V = np.concatenate([vp.reshape(b, hkv, past, d)[:, :, :7], vn.reshape(b, hkv, 1, d)], axis=2).astype(np.float64)
    want = np.zeros((b, h, d))
    for bi in range(b):
        for hi in range(h):
            s = K[bi, hi // 2] @ Q[bi, hi] / math.sqrt(d)
            p = np.exp(s - s.max())
            want[bi, hi] = (p / p.sum()) @ V[bi, hi // 2]
    assert np.max(np.abs(got.reshape(b, h, d) - want)) < 1e-5


def test_matmul_is_an_ascending_fma_chain_then_truncation():
    m, k, n = 3, 37, 16
    rng = np.random.default_rng(7)
    a = orc.f32_to_bf16_rne(rng.standard_normal(m * k).astype(np.float32))
    b = orc.f32_to_bf16_rne(rng.standard_normal(k * n).astype(np.float32))
    got = orc.matmul(a, b, m, k, n, kc.DTYPE_BF16)
    A, B = orc.bf16_to_f32(a).reshape(m, k), orc.bf16_to_f32(b).reshape(k, n)
    want = np.zeros((m, n), dtype=np.float32)
    for i in range(m):
        for j in range(n):
            acc = np.float32(0)
            for kk in range(k):
                acc = np.float32(math.fma(float(A[i, kk]), float(B[kk, j]), float(acc))) if hasattr(math, "fma") else acc
            want[i, j] = acc
    if hasattr(math, "fma"):
        assert np.array_equal(got.reshape(m, n), orc.f32_to_bf16_trunc(want).reshape(m, n))
    # f64 reference bound of the reference's conformance test (tests/conformance.rs:256): 8e-3
    ref = A.astype(np.float64) @ B.astype(np.float64)
    err = np.max(np.abs(orc.bf16_to_f32(got).reshape(m, n) - ref)) / np.max(np.abs(ref))
    assert err <= 8e-3


def test_fused_epilogues_equal_the_unfused_pair():
    # float_kernels.rs:822-891: narrow, re-widen, epilogue, narrow
    m, k, n = 4, 32, 24
    rng = np.random.default_rng(11)
    a = orc.f32_to_bf16_rne(rng.standard_normal(m * k).astype(np.float32))
    b = orc.f32_to_bf16_rne(rng.standard_normal(k * n).astype(np.float32))
    r = orc.f32_to_bf16_rne(rng.standard_normal(m * n).astype(np.float32))
    plain = orc.matmul(a, b, m, k, n, kc.DTYPE_BF16)
    assert np.array_equal(orc.matmul(a, b, m, k, n, kc.DTYPE_BF16, act=kc.FUSED_SILU),
                          orc.unary_lut(kc.LUT_SILU, kc.DTYPE_BF16, plain))
    assert np.array_equal(orc.matmul(a, b, m, k, n, kc.DTYPE_BF16, residual=r),
                          orc.binary(0, plain, r, kc.DTYPE_BF16))


def test_kv_cache_write_ring():
    # cpu/kernels.rs:455-501; tests/kv_cache_write.rs:126-156 (wrap-around)
    planes, bucket, new_rows, row = 2, 5, 2, 3
    cache = np.arange(planes * bucket * row, dtype=np.uint8)
    new = 200 + np.arange(planes * new_rows * row, dtype=np.uint8)
    rc, out = orc.kv_cache_write(cache, new, 4 + 5 * 3, planes, bucket, new_rows, row)   # pos wraps to 4
    assert rc == 0
    o = out.reshape(planes, bucket, row)
    n = new.reshape(planes, new_rows, row)
    assert np.array_equal(o[:, 4], n[:, 0]) and np.array_equal(o[:, 0], n[:, 1])
    assert np.array_equal(o[:, 1:4], cache.reshape(planes, bucket, row)[:, 1:4])
    assert orc.kv_cache_write(cache, new, 0, planes, 0, new_rows, row)[0] == -3
    assert orc.kv_cache_write(cache, new, 0, planes, 1, 2, row)[0] == -3


def test_add_rms_norm_and_transpose_restatements():
    # AddRmsNorm = RmsNorm over the f32 sum x + residual (cpu/float_kernels.rs:1656-1679); with the
    # residual folded into x beforehand in f32 the two restatements must agree bit for bit
    rng = np.random.default_rng(9)
    x, r = rng.standard_normal((2, 6 * 50)).astype(np.float32)
    g = rng.standard_normal(50).astype(np.float32)
    eps = struct.unpack("<I", struct.pack("<f", 1e-5))[0]
    a = orc.add_rms_norm(x, r, g, 6, 50, eps, kc.DTYPE_F32)
    b = orc.rms_norm(x + r, g, 6, 50, eps, kc.DTYPE_F32)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.array_equal(orc.add_rms_norm(x, None, g, 6, 50, eps, kc.DTYPE_F32).view(np.uint32),
                          orc.rms_norm(x, g, 6, 50, eps, kc.DTYPE_F32).view(np.uint32))
    # Transpose: output axis i is input axis perm[i] (cpu/float_kernels.rs:2980-3027)
    t = np.arange(2 * 3 * 4 * 5, dtype=np.uint16)
    for perm in ((0, 1, 2, 3), (3, 2, 1, 0), (1, 3, 0, 2)):
        got = orc.transpose(t, (2, 3, 4, 5), perm, 2).view(np.uint16)
        assert np.array_equal(got, np.transpose(t.reshape(2, 3, 4, 5), perm).reshape(-1))


def test_softmax_restatement_meets_the_reference_pins():
    # crates/hologram-compute/tests/pinned_semantics.rs:193-217: a fully masked row is +0.0 everywhere, the
    # finite sibling row is untouched; tests/conformance.rs:305-335: within 1e-4 of the f64 softmax at
    # these shapes and every row sums to 1 within 1e-3
    f = 5
    rows = np.concatenate([np.full(f, -np.inf, np.float32), np.random.default_rng(9).standard_normal(f).astype(np.float32)])
    sm = orc.softmax(rows, 2, f, kc.DTYPE_F32)
    assert np.array_equal(sm[:f].view(np.uint32), np.zeros(f, np.uint32)) and np.all(np.isfinite(sm[f:]))
    for idx, (b, feat) in enumerate(((1, 4), (8, 31), (16, 128), (4, 1024))):
        x = (np.random.default_rng(0x300 + idx).random(b * feat, dtype=np.float32) * 2 - 1) * 4
        got = orc.softmax(x, b, feat, kc.DTYPE_F32).reshape(b, feat)
        x64 = x.astype(np.float64).reshape(b, feat)
        e = np.exp(x64 - x64.max(axis=1, keepdims=True))
        assert np.max(np.abs(got - e / e.sum(axis=1, keepdims=True))) < 1e-4
        assert np.all(np.abs(got.sum(axis=1) - 1.0) < 1e-3)


def test_layer_norm_restatement_meets_the_reference_pins():
    # crates/hologram-compute/tests/conformance.rs:336-395: within 1e-3 of the f64 layer norm at these shapes;
    # tests/pinned_semantics.rs:245-275: the declared epsilon is authoritative, 0 selects 1e-9
    eps = np.float32(1e-5)
    bits = int(eps.view(np.uint32))
    for idx, (b, f) in enumerate(((2, 8), (8, 33), (16, 256))):
        rng = np.random.default_rng(0x400 + idx)
        x, g, bt = (rng.standard_normal(n).astype(np.float32) for n in (b * f, f, f))
        got = orc.layer_norm(x, g, bt, b, f, bits, kc.DTYPE_F32).reshape(b, f)
        x64 = x.astype(np.float64).reshape(b, f)
        mean = x64.mean(axis=1, keepdims=True)
        var = ((x64 - mean) ** 2).mean(axis=1, keepdims=True)
        want = (x64 - mean) / np.sqrt(var + float(eps)) * g.astype(np.float64) + bt.astype(np.float64)
        assert np.max(np.abs(got - want)) < 1e-3
    x = (np.float32(1.0) + np.arange(8, dtype=np.float32) * np.float32(1e-7)).astype(np.float32)
    e12 = orc.layer_norm(x, None, None, 1, 8, int(np.float32(1e-12).view(np.uint32)), kc.DTYPE_F32)
    e9 = orc.layer_norm(x, None, None, 1, 8, int(np.float32(1e-9).view(np.uint32)), kc.DTYPE_F32)
    dflt = orc.layer_norm(x, None, None, 1, 8, 0, kc.DTYPE_F32)
    assert not np.array_equal(e12.view(np.uint32), e9.view(np.uint32))
    assert np.array_equal(dflt.view(np.uint32), e9.view(np.uint32))


def test_broadcast_restatement_equals_numpy_broadcasting():
    # expand_float / broadcast_binary_float (cpu/float_kernels.rs:3405-3444, :3250-3397): stride 0 on the
    # size-1 axes of the small operand; one f32 operation per element
    rng = np.random.default_rng(112)
    in_dims, out_dims = (1, 5, 1, 7), (3, 5, 4, 7)
    small = rng.standard_normal(int(np.prod(in_dims))).astype(np.float32)
    other = rng.standard_normal(int(np.prod(out_dims))).astype(np.float32)
    s4, o4 = small.reshape(in_dims), other.reshape(out_dims)
    assert np.array_equal(orc.broadcast(small, None, in_dims, out_dims, 4).view(np.float32).reshape(out_dims), np.broadcast_to(s4, out_dims))
    for op, fn in ((0, np.add), (1, np.subtract), (2, np.multiply)):
        for lhs in (True, False):
            want = fn(s4, o4) if lhs else fn(o4, s4)
            got = orc.broadcast(small, other, in_dims, out_dims, 4, op, lhs, kc.DTYPE_F32).view(np.float32).reshape(out_dims)
            assert np.array_equal(got.view(np.uint32), want.astype(np.float32).view(np.uint32))


def test_reduce_restatement_equals_numpy_on_exact_cases():
    # reduce_float (cpu/float_kernels.rs:1901-2022): min / max are order-free, small-integer sums and
    # products are exact in f32, so numpy gives the expected bits; keepdims layout = reduced axes dropped
    rng = np.random.default_rng(55)
    dims = (3, 4, 5, 2)
    x = rng.integers(-4, 5, size=int(np.prod(dims))).astype(np.float32)
    x4 = x.reshape(dims)
    for mask, axes in ((0b0010, (1,)), (0b1010, (1, 3)), (0b0101, (0, 2)), (0, (0, 1, 2, 3)), (0b1111, (0, 1, 2, 3))):
        for kind, fn in ((0, np.sum), (2, np.min), (3, np.max)):
            got = orc.reduce(x, dims, mask, kind, False, kc.DTYPE_F32)
            assert np.array_equal(got, fn(x4, axis=axes).astype(np.float32).reshape(-1))
        got = orc.reduce(x, dims, mask, 0, True, kc.DTYPE_F32)
        cnt = int(np.prod([dims[a] for a in axes]))
        assert np.array_equal(got, (np.sum(x4, axis=axes).astype(np.float32) * (np.float32(1.0) / np.float32(cnt))).reshape(-1))
    p = rng.integers(1, 3, size=24).astype(np.float32)
    assert np.array_equal(orc.reduce(p, (2, 3, 4), 0b010, 1, False, kc.DTYPE_F32), np.prod(p.reshape(2, 3, 4), axis=1).reshape(-1))


def test_exact_elementwise_restatement_on_known_answers():
    # cpu/float_kernels.rs:3446-3500, :3660-3733: IEEE division by zero, floored modulo whose sign follows
    # the divisor, half-away-from-zero rounding, NaN-ignoring min / max, comparisons as 1.0 / 0.0
    f = lambda *v: np.array(v, dtype=np.float32)
    e = lambda tag, a, b=None: orc.elementwise(tag, a, b, kc.DTYPE_F32)
    assert np.array_equal(e(kc.K_DIV, f(1, -1, 6), f(0, 0, 4)), f(np.inf, -np.inf, 1.5))
    assert np.isnan(e(kc.K_DIV, f(0), f(0))[0]) and np.isnan(e(kc.K_MOD, f(1), f(0))[0])
    assert np.array_equal(e(kc.K_MOD, f(5, -5, 5, -5), f(3, 3, -3, -3)), f(2, 1, -1, -2))
    assert np.array_equal(e(kc.K_ROUND, f(0.5, -0.5, 1.5, 2.5, -2.5)), f(1, -1, 2, 3, -3))
    assert np.array_equal(e(kc.K_MIN, f(np.nan, 1, 2), f(3, np.nan, 1)), f(3, 1, 1))
    assert np.array_equal(e(kc.K_MAX, f(np.nan, 1, 2), f(3, np.nan, 1)), f(3, 1, 2))
    assert np.array_equal(e(kc.K_RELU, f(-1, 2, np.nan)), f(0, 2, 0))
    assert np.array_equal(e(kc.K_SIGN, f(-3, 0, 7, np.nan)), f(-1, 0, 1, 0))
    assert np.array_equal(e(kc.K_IS_NAN, f(np.nan, 1)), f(1, 0))
    assert np.array_equal(e(kc.K_LESS_OR_EQUAL, f(1, 2, np.nan), f(1, 1, 1)), f(1, 0, 0))
    assert np.array_equal(e(kc.K_SQRT, f(4, 2)), np.sqrt(f(4, 2))) and np.array_equal(e(kc.K_RECIPROCAL, f(4, 0)), f(0.25, np.inf))


def test_legacy_attention_restatement_meets_the_reference_conformance_cases():
    # crates/hologram-compute/tests/conformance.rs:778-935 (kc8c): causal, grouped-query and explicit-scale cases
    # against a float64 attention, 1e-4
    from helpers import ATTENTION_CASES, attention_f64
    for idx, (b, h, hkv, s, d, causal, mult) in enumerate(ATTENTION_CASES):
        rng = np.random.default_rng(0x8c0 + idx)
        q, k, v = (rng.standard_normal(n).astype(np.float32) for n in (b * h * s * d, b * hkv * s * d, b * hkv * s * d))
        bits = int(np.float32(mult).view(np.uint32)) if mult else 0
        got = orc.attention(q, k, v, b, h, hkv if hkv != h else 0, s, d, causal, bits, kc.DTYPE_F32)
        assert np.max(np.abs(got - attention_f64(q, k, v, b, h, hkv, s, d, causal, mult))) < 1e-4


def test_dequant_activation_restatement_is_the_unfused_composition():
    # crates/hologram-compute/tests/dequant_activation.rs:66-140: over every i8 code (scale 0.05, zero point -7)
    # the fused table is bit-identical to Dequantize (-> f32) followed by the scalar activation
    codes = np.arange(256, dtype=np.uint8)
    scale, zp = np.float32(0.05), -7
    for act in (kc.LUT_GELU, kc.LUT_SILU, kc.LUT_SIGMOID, kc.LUT_TANH):
        fused = orc.dequant_activation(codes, 256, kc.DTYPE_I8, act, scale, zp)
        deq = orc.dequantize(codes.view(np.int8), None, None, 0, 0, float(scale), zp, kc.DTYPE_F32)
        unfused = np.array([orc.lib.holo_or_act(act, float(v)) for v in deq], dtype=np.float32)
        assert np.array_equal(fused.view(np.uint32), unfused.view(np.uint32))
    # i4: two signed nibbles per byte, low nibble first
    packed = np.array([0x80 | 0x07, 0xF1], dtype=np.uint8)          # 7, -8, 1, -1
    got = orc.dequant_activation(packed, 4, kc.DTYPE_I4, kc.LUT_SIGMOID, np.float32(0.5), 0)
    want = np.array([orc.lib.holo_or_act(kc.LUT_SIGMOID, float(np.float32(q) * np.float32(0.5))) for q in (7, -8, 1, -1)], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_quantized_weight_tier_restatements_reproduce_the_reference_goldens():
    # crates/hologram-compute/src/cpu/simd.rs:8236-8281: the FNV-1a-64 of the output bits of the three
    # output-major decode products (i8, packed i4, E8 codebook) on the reference's fixed operands
    m, k, n = 3, 64, 24
    a = (np.array([float(i * 37 % 91) for i in range(m * k)], dtype=np.float32) - np.float32(45.0)) * np.float32(0.031)
    scales = np.float32(0.011) + np.arange(n, dtype=np.float32) * np.float32(0.0007)
    bq = np.array([(i * 31 % 255) - 127 for i in range(k * n)], dtype=np.int8)
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))["fnv1a64_of_output_bits"]
    assert orc.fnv1a64_f32(orc.matmul_w8a8_omajor(a, bq, scales, m, k, n)) == int(golden["i8_w8a8"], 16)
    bq4 = np.array([(i * 53 + 9) % 251 for i in range(k * n // 2)], dtype=np.uint8)
    assert orc.fnv1a64_f32(orc.matmul_w8a8_omajor(a, bq4, scales, m, k, n, i4=True)) == int(golden["i4_w4a8"], 16)
    cb = np.array([(i * 37 + 11) % 255 - 127 for i in range(256 * 8)], dtype=np.int8)
    bq8 = np.array([(i * 17 + 3) % 256 for i in range(n * (k // 8))], dtype=np.uint8)
    assert orc.fnv1a64_f32(orc.matmul_w8a8_omajor(a, bq8, scales, m, k, n, codebook=cb)) == int(golden["e8cb_w1a8"], 16)


def test_mask_form_restatement_equals_scalar_form_bitwise():
    # the reference pins that a realized-length mask reproduces DecodeAttentionValid bit for bit
    # (crates/hologram-compute/tests/decode_attention_valid.rs:226-282); all-erased row = zeros
    b, h, kv, past, d = 2, 4, 2, 19, 24
    rng = np.random.default_rng(12)
    arrs = [rng.standard_normal(n).astype(np.float32) for n in (b * h * d, b * kv * past * d, b * kv * past * d, b * kv * d, b * kv * d)]
    for valid in (0, 7, 19):
        mask = np.zeros((1, past + 1), np.float32)
        mask[0, valid:past] = -np.inf
        a = orc.decode_attention_mask(*arrs, mask, b, h, kv, 1, past, 1, d, 0, kc.DTYPE_F32)
        rc, v = orc.decode_attention_valid(*arrs, valid, b, h, kv, 1, past, 1, d, 0, kc.DTYPE_F32)
        assert rc == 0 and np.array_equal(a.view(np.uint32), v.view(np.uint32))
    mask = np.full((1, past + 1), -np.inf, np.float32)
    z = orc.decode_attention_mask(*arrs, mask, b, h, kv, 1, past, 1, d, 0, kc.DTYPE_F32)
    assert not np.any(z)


def test_kn_dequant_matmul_restatement_against_the_naive_loop():
    # crates/hologram-compute/src/cpu/simd.rs:7175-7204 (matmul_i8_per_channel_matches_naive): the fused per-channel kernel
    # within 1e-4 (relative, floor 1) of the naive multiply-add loop with the scale applied at the end, on the
    # reference's four shapes and value laws
    for m, k, n in ((1, 64, 48), (3, 17, 33), (5, 9, 16), (1, 2048, 64)):
        a = (((np.arange(m * k) % 13).astype(np.float32)) - np.float32(6.0)) * np.float32(0.1)
        bq = ((np.arange(k * n, dtype=np.int64) % 255) - 127).astype(np.int8)
        scales = np.float32(0.01) + np.arange(n, dtype=np.float32) * np.float32(0.001)
        got = orc.matmul_dequant_kn(a, bq, m, k, n, kc.DTYPE_I8, scales, np.zeros(n, dtype=np.int32), channels=n, inner=1)
        want = (a.reshape(m, k).astype(np.float64) @ bq.reshape(k, n).astype(np.float64)) * scales.astype(np.float64)
        err = np.abs(got.reshape(m, n) - want) / np.maximum(np.abs(want), 1.0)
        assert err.max() < 1e-4
    # the two definitions factor the scale differently: with nonzero zero points the weight is dequantized first
    rng = np.random.default_rng(0)
    m, k, n = 2, 64, 16
    a = rng.standard_normal(m * k).astype(np.float32)
    bq = rng.integers(-127, 128, size=k * n, dtype=np.int8)
    sc = (rng.random(n, dtype=np.float32) * np.float32(0.02) + np.float32(0.001)).astype(np.float32)
    zp = rng.integers(-3, 4, size=n, dtype=np.int32)
    got = orc.matmul_dequant_kn(a, bq, m, k, n, kc.DTYPE_I8, sc, zp, channels=n, inner=1)
    deq = ((bq.reshape(k, n).astype(np.int32) - zp[None, :]).astype(np.float32) * sc[None, :]).astype(np.float32)
    assert np.array_equal(got.view(np.uint32), orc.matmul(a, deq.reshape(-1), m, k, n, kc.DTYPE_F32).view(np.uint32))


def test_matmul_add_activation_restatement_is_the_unfused_f32_triple():
    # session.rs:2220-2226: for f32 the triple is bit-identical to the three separate calls (no narrowing to skip)
    rng = np.random.default_rng(5)
    m, k, n = 4, 40, 24
    a, b, r = (rng.standard_normal(c, dtype=np.float32) for c in (m * k, k * n, m * n))
    got = orc.matmul_add_activation(a, b, r, m, k, n, kc.DTYPE_F32, kc.FUSED_GELU)
    s = orc.matmul(a, b, m, k, n, kc.DTYPE_F32) + r
    want = np.array([orc.lib.holo_or_act(kc.LUT_GELU, float(v)) for v in s], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
