"""Decoder glue ops on the GPU against the oracle (through the C ABI)."""
import struct

import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc
from helpers import norm_max_err, synth_bf16

pytestmark = pytest.mark.gpu
BF = kc.DTYPE_BF16


def f32bits(x):
    return struct.unpack("<I", struct.pack("<f", x))[0]


def test_add_mul_bit_exact(backend):
    n = 64 * 4096 + 3
    a, b = synth_bf16(n, 1.0, 1), synth_bf16(n, 2.0, 2)
    for op, ctor in ((0, kc.KernelCall.Add), (1, kc.KernelCall.Mul)):
        ws = hb.DeviceWorkspace(backend, 3)
        ws.put(0, a)
        ws.put(1, b)
        ws.alloc(2, n * 2)
        backend.dispatch(ctor(kc.BinaryCall(kc.rb(0), kc.rb(1), kc.rb(2), n, 16, BF)), ws)
        assert np.array_equal(ws.read(2, n * 2, np.uint16), orc.binary(op, a, b, BF))
    # f32 form
    af, bf_ = np.random.default_rng(0).standard_normal((2, 1000)).astype(np.float32)
    ws = hb.DeviceWorkspace(backend, 3)
    ws.put(0, af)
    ws.put(1, bf_)
    ws.alloc(2, af.nbytes)
    backend.dispatch(kc.KernelCall.Add(kc.BinaryCall(kc.rb(0), kc.rb(1), kc.rb(2), af.size, 32, kc.DTYPE_F32)), ws)
    assert np.array_equal(ws.read(2, af.nbytes, np.float32), af + bf_)


def test_rms_norm_within_tolerance(backend):
    batch, feature = 64, 4096
    x, g = synth_bf16(batch * feature, 1.5, 3), synth_bf16(feature, 1.0, 4)
    ws = hb.DeviceWorkspace(backend, 3)
    ws.put(0, x)
    ws.put(1, g)
    ws.alloc(2, x.nbytes)
    call = kc.NormCall(kc.rb(0), kc.rb(1), kc.NONE, kc.NONE, kc.rb(2), batch, feature, 0, 0, f32bits(1e-5), BF)
    backend.dispatch(kc.KernelCall.RmsNorm(call), ws)
    got = orc.bf16_to_f32(ws.read(2, x.nbytes, np.uint16))
    want = orc.bf16_to_f32(orc.rms_norm(x, g, batch, feature, f32bits(1e-5), BF))
    # the sum of squares is reduced in parallel: a 1-ulp bf16 difference is allowed
    assert norm_max_err(got, want) <= 1e-2
    assert np.mean(got.view(np.uint32) == want.view(np.uint32)) > 0.99
    bad = kc.NormCall(kc.rb(0), kc.rb(1), kc.NONE, kc.NONE, kc.rb(2), batch, feature, 0, 0, f32bits(-1.0), BF)
    with pytest.raises(hb.BackendError) as e:
        backend.dispatch(kc.KernelCall.RmsNorm(bad), ws)
    assert e.value.variant == "UnsupportedOp"


def test_rope_bit_exact(backend):
    n, d = 64 * 32 * 128, 128
    x, c, s = synth_bf16(n, 1.0, 5), synth_bf16(n, 0.7, 6), synth_bf16(n, 0.7, 7)
    ws = hb.DeviceWorkspace(backend, 4)
    for i, v in enumerate((x, c, s)):
        ws.put(i, v)
    ws.alloc(3, x.nbytes)
    backend.dispatch(kc.KernelCall.RotaryEmbedding(kc.RoPECall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), d, n, BF)), ws)
    assert np.array_equal(ws.read(3, x.nbytes, np.uint16), orc.rope(x, c, s, d, BF))
    with pytest.raises(hb.BackendError):
        backend.dispatch(kc.KernelCall.RotaryEmbedding(kc.RoPECall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), 7, n, BF)), ws)


def test_gather_embedding_rows(backend):
    vocab, dm, k = 1000, 256, 64
    data = synth_bf16(vocab * dm, 1.0, 8)
    idx = np.random.default_rng(9).integers(-vocab, vocab, size=k).astype(np.int32)
    ws = hb.DeviceWorkspace(backend, 3)
    ws.put(0, data)
    ws.put(1, idx)
    ws.alloc(2, k * dm * 2)
    call = kc.GatherCall(kc.rb(0), kc.rb(1), kc.rb(2), 1, vocab, dm, k, kc.DTYPE_I32, BF)
    backend.dispatch(kc.KernelCall.Gather(call), ws)
    rc, want = orc.gather(data, idx, 1, vocab, dm, BF)
    assert rc == 0 and np.array_equal(ws.read(2, k * dm * 2, np.uint16), want)
    # out-of-range index fails loud at the next synchronising call
    idx[3] = vocab
    ws.write(1, idx)
    backend.dispatch(kc.KernelCall.Gather(call), ws)
    with pytest.raises(hb.BackendError) as e:
        backend.synchronize()
    assert e.value.variant == "SlotOutOfRange"
    backend.synchronize()


def test_cast_and_dequantize(backend):
    n = 10007
    x = synth_bf16(n, 3.0, 10)
    ws = hb.DeviceWorkspace(backend, 4)
    ws.put(0, x)
    ws.alloc(1, n * 4)
    backend.dispatch(kc.KernelCall.Cast(kc.CastCall(kc.rb(0), kc.rb(1), n, BF, kc.DTYPE_F32)), ws)
    f = ws.read(1, n * 4, np.float32)
    assert np.array_equal(f.view(np.uint32), orc.bf16_to_f32(x).view(np.uint32))
    ws.alloc(2, n * 2)
    backend.dispatch(kc.KernelCall.Cast(kc.CastCall(kc.rb(1), kc.rb(2), n, kc.DTYPE_F32, kc.DTYPE_F16)), ws)
    assert np.array_equal(ws.read(2, n * 2, np.uint16), orc.cast_float(f, kc.DTYPE_F32, kc.DTYPE_F16))
    # per-row dequantize: channels = rows, inner = d, zero-point 0
    rows, d = 37, 128
    rng = np.random.default_rng(11)
    codes = rng.integers(-127, 128, size=rows * d).astype(np.int8)
    scales = rng.random(rows).astype(np.float32)
    zps = np.zeros(rows, dtype=np.int32)
    ws2 = hb.DeviceWorkspace(backend, 4)
    ws2.put(0, codes)
    ws2.put(1, scales)
    ws2.put(2, zps)
    ws2.alloc(3, rows * d * 4)
    call = kc.DequantizeCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), rows * d, rows, d, kc.DTYPE_I8, kc.DTYPE_F32, 0, 0)
    backend.dispatch(kc.KernelCall.Dequantize(call), ws2)
    want = orc.dequantize(codes, scales, zps, rows, d, 0.0, 0, kc.DTYPE_F32)
    assert np.array_equal(ws2.read(3, rows * d * 4, np.float32).view(np.uint32), want.view(np.uint32))


def test_kv_cache_write_copy_and_in_place(backend):
    planes, bucket, new_rows, row = 16, 40, 3, 128
    rng = np.random.default_rng(12)
    cache = rng.integers(0, 256, size=planes * bucket * row).astype(np.uint8)
    new = rng.integers(0, 256, size=planes * new_rows * row).astype(np.uint8)
    for pos in (0, 17, 38, 39, 4000000001):
        rc, want = orc.kv_cache_write(cache, new, pos % (1 << 32), planes, bucket, new_rows, row)
        ws = hb.DeviceWorkspace(backend, 4)
        ws.put(0, cache)
        ws.put(1, new)
        ws.put(2, np.array([pos % (1 << 32)], dtype=np.uint32))
        ws.alloc(3, cache.nbytes)
        call = kc.KvCacheWriteCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), planes, bucket, new_rows, row)
        backend.dispatch(kc.KernelCall.KvCacheWrite(call), ws)
        assert np.array_equal(ws.read(3, cache.nbytes), want)
        # in-place move form (cache == output): same bytes, O(new_rows) work
        call2 = kc.KvCacheWriteCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(0), planes, bucket, new_rows, row)
        backend.dispatch(kc.KernelCall.KvCacheWrite(call2), ws)
        assert np.array_equal(ws.read(0, cache.nbytes), want)
    with pytest.raises(hb.BackendError) as e:
        bad = kc.KvCacheWriteCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), planes, 2, 3, row)
        backend.dispatch(kc.KernelCall.KvCacheWrite(bad), ws)
    assert e.value.variant == "UnsupportedOp"


@pytest.mark.parametrize("dtype,d", [(kc.DTYPE_BF16, 128), (kc.DTYPE_BF16, 96), (kc.DTYPE_F32, 64), (kc.DTYPE_F16, 256)])
def test_quantize_rows_bit_exact(backend, dtype, d):
    rows = 4099
    rng = np.random.default_rng(d)
    x = rng.standard_normal(rows * d).astype(np.float32)
    x.reshape(rows, d)[5] = 0.0                      # all-zero row
    x.reshape(rows, d)[6, 3] = np.inf                # inf row
    x.reshape(rows, d)[7, 1] = np.nan                # NaN element is skipped by the max scan
    x.reshape(rows, d)[8] *= 1e-30
    if dtype == kc.DTYPE_BF16:
        xs = orc.f32_to_bf16_rne(x)
    elif dtype == kc.DTYPE_F16:
        xs = x.astype(np.float16).view(np.uint16)
    else:
        xs = x
    ws = hb.DeviceWorkspace(backend, 3)
    ws.put(0, xs)
    ws.alloc(1, rows * d)
    ws.alloc(2, rows * 4)
    backend.dispatch(kc.KernelCall.QuantizeRowsI8(kc.QuantizeRowsI8Call(kc.rb(0), kc.rb(1), kc.rb(2), rows, d, dtype)), ws)
    codes, scales = orc.quantize_rows_i8(xs, dtype, rows, d)
    assert np.array_equal(ws.read(1, rows * d, np.int8), codes)
    assert np.array_equal(ws.read(2, rows * 4, np.uint32), scales.view(np.uint32))


def test_add_rms_norm_within_tolerance(backend):
    # AddRmsNorm (cpu/float_kernels.rs:1567-1681): the norm of x + residual, the sum kept in f32
    for batch, feature, dt in ((64, 4096, BF), (5, 100, BF), (3, 257, kc.DTYPE_F32)):
        if dt == BF:
            x, r, g = synth_bf16(batch * feature, 1.5, 30), synth_bf16(batch * feature, 0.7, 31), synth_bf16(feature, 1.0, 32)
        else:
            rng = np.random.default_rng(5)
            x, r = rng.standard_normal((2, batch * feature)).astype(np.float32)
            g = rng.standard_normal(feature).astype(np.float32)
        ws = hb.DeviceWorkspace(backend, 4)
        ws.put(0, x)
        ws.put(1, g)
        ws.put(2, r)
        ws.alloc(3, x.nbytes)
        call = kc.NormCall(kc.rb(0), kc.rb(1), kc.NONE, kc.rb(2), kc.rb(3), batch, feature, 0, 0, f32bits(1e-5), dt)
        backend.dispatch(kc.KernelCall.AddRmsNorm(call), ws)
        want = orc.add_rms_norm(x, r, g, batch, feature, f32bits(1e-5), dt)
        if dt == BF:
            got, want = orc.bf16_to_f32(ws.read(3, x.nbytes, np.uint16)), orc.bf16_to_f32(want)
            assert norm_max_err(got, want) <= 1e-2
            assert np.mean(got.view(np.uint32) == want.view(np.uint32)) > 0.99
        else:
            assert norm_max_err(ws.read(3, x.nbytes, np.float32), want) <= 1e-5
        # without the residual operand it is RmsNorm
        call = kc.NormCall(kc.rb(0), kc.rb(1), kc.NONE, kc.NONE, kc.rb(3), batch, feature, 0, 0, f32bits(1e-5), dt)
        backend.dispatch(kc.KernelCall.AddRmsNorm(call), ws)
        plain = orc.rms_norm(x, g, batch, feature, f32bits(1e-5), dt)
        view = np.uint16 if dt == BF else np.float32
        got = ws.read(3, x.nbytes, view)
        if dt == BF:
            assert norm_max_err(orc.bf16_to_f32(got), orc.bf16_to_f32(plain)) <= 1e-2
        else:
            assert norm_max_err(got, plain) <= 1e-5


@pytest.mark.parametrize("dims,perm,dt", [
    ((64, 32, 128), (1, 0, 2), kc.DTYPE_BF16),       # [tokens, heads, d] -> [heads, tokens, d]
    ((7, 5), (1, 0), kc.DTYPE_F32),
    ((2, 3, 4, 5), (3, 1, 0, 2), kc.DTYPE_I8),
    ((3, 1, 4, 1, 5, 2, 2, 3), (7, 0, 6, 1, 5, 2, 4, 3), kc.DTYPE_I64),
    ((11,), (0,), kc.DTYPE_BF16),
])
def test_transpose_bit_exact(backend, dims, perm, dt):
    es = {kc.DTYPE_BF16: 2, kc.DTYPE_F32: 4, kc.DTYPE_I8: 1, kc.DTYPE_I64: 8}[dt]
    total = int(np.prod(dims))
    x = np.random.default_rng(total).integers(0, 256, total * es, dtype=np.uint8)
    ws = hb.DeviceWorkspace(backend, 2)
    ws.put(0, x)
    ws.alloc(1, x.nbytes)
    backend.dispatch(kc.KernelCall.Transpose(kc.TransposeCall.make(kc.rb(0), kc.rb(1), dims, perm, dt)), ws)
    got = ws.read(1, x.nbytes)
    assert np.array_equal(got, orc.transpose(x, dims, perm, es))
    # independent check against numpy's own transpose
    ref = np.transpose(x.reshape(*dims, es), list(perm) + [len(dims)]).reshape(-1)
    assert np.array_equal(got, ref)


def test_transpose_refusals(backend):
    ws = hb.DeviceWorkspace(backend, 2)
    ws.alloc(0, 64)
    ws.alloc(1, 64)
    with pytest.raises(hb.BackendError) as e:   # not a permutation
        backend.dispatch(kc.KernelCall.Transpose(kc.TransposeCall.make(kc.rb(0), kc.rb(1), (2, 3), (0, 0), BF)), ws)
    assert e.value.variant == "UnsupportedOp"
    with pytest.raises(hb.BackendError) as e:   # output too short
        backend.dispatch(kc.KernelCall.Transpose(kc.TransposeCall.make(kc.rb(0), kc.rb(1), (8, 8), (1, 0), BF)), ws)
    assert e.value.variant == "SlotOutOfRange"


def test_slice_and_concat_are_byte_placement(backend):
    # Slice: a contiguous copy whose start is the input ref's offset (cpu/kernels.rs:688-700);
    # Concat: out = a || b at the refs' extents (cpu/float_kernels.rs:2963-2974)
    a = synth_bf16(1000, 1.0, 40)
    b = synth_bf16(300, 1.0, 41)
    ws = hb.DeviceWorkspace(backend, 4)
    ws.put(0, a)
    ws.put(1, b)
    ws.alloc(2, 4096)
    ws.alloc(3, 4096)
    backend.dispatch(kc.KernelCall.Slice(kc.LayoutCall(kc.rb(0, 200, 0), kc.rb(2), 400, BF)), ws)
    assert np.array_equal(ws.read(kc.rb(2, 0, 800), dtype=np.uint16), a[100:500])
    backend.dispatch(kc.KernelCall.Concat(kc.BinaryCall(kc.rb(0, 0, 2000), kc.rb(1, 0, 600), kc.rb(3), 1300, 16, BF)), ws)
    assert np.array_equal(ws.read(kc.rb(3, 0, 2600), dtype=np.uint16), np.concatenate([a, b]))
    # an output shorter than a || b is refused against the output slot
    ws.alloc(3, 1024)
    with pytest.raises(hb.BackendError) as e:
        backend.dispatch(kc.KernelCall.Concat(kc.BinaryCall(kc.rb(0, 0, 2000), kc.rb(1, 0, 600), kc.rb(3), 1300, 16, BF)), ws)
    assert e.value.variant == "SlotOutOfRange" and e.value.slot == 3


def test_rope_quantize_rows_is_the_pair_bit_for_bit(backend):
    # extension 0x8004: RotaryEmbedding then QuantizeRowsI8 of its rows (the K path of a decoder layer)
    rows, d = 64 * 8, 128
    n = rows * d
    x, c, s = synth_bf16(n, 1.0, 50), synth_bf16(n, 0.7, 51), synth_bf16(n, 0.7, 52)
    x[: d] = 0                                     # an all-zero head: zero codes, scale 0
    ws = hb.DeviceWorkspace(backend, 6)
    for i, a in enumerate((x, c, s)):
        ws.put(i, a)
    ws.alloc(3, n * 2)
    ws.alloc(4, n)
    ws.alloc(5, rows * 4)
    call = kc.RopeQuantizeCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), rows, d, BF)
    backend.dispatch(kc.KernelCall.RopeQuantizeRowsI8(call), ws)
    rot = orc.rope(x, c, s, d, BF)
    codes, scales = orc.quantize_rows_i8(rot, BF, rows, d)
    assert np.array_equal(ws.read(3, n * 2, np.uint16), rot)
    assert np.array_equal(ws.read(4, n, np.int8), codes)
    assert np.array_equal(ws.read(5, rows * 4, np.float32).view(np.uint32), scales.view(np.uint32))


def test_softmax_rows(backend):
    # softmax_float (cpu/float_kernels.rs:1758-1875); the parallel sum differs from the CPU's
    # left-to-right sum by rounding only
    for batch, feature, dt in ((64, 4096, kc.DTYPE_F32), (7, 33, kc.DTYPE_F32), (32, 1000, BF)):
        rng = np.random.default_rng(feature)
        x = (rng.standard_normal(batch * feature) * 3).astype(np.float32)
        x[:feature] = -np.inf                       # an impossible distribution: exactly zero everywhere
        x[feature + 3] = -np.inf
        xin = x if dt == kc.DTYPE_F32 else orc.f32_to_bf16_rne(x)
        ws = hb.DeviceWorkspace(backend, 2)
        ws.put(0, xin)
        ws.alloc(1, xin.nbytes)
        backend.dispatch(kc.KernelCall.Softmax(kc.SoftmaxCall(kc.rb(0), kc.rb(1), batch, feature, dt)), ws)
        want = orc.softmax(xin, batch, feature, dt)
        if dt == kc.DTYPE_F32:
            got = ws.read(1, xin.nbytes, np.float32)
            assert not got[:feature].any() and got[feature + 3] == 0.0
            assert np.allclose(got, want, rtol=2e-5, atol=1e-12)   # the reference's own bound is 1e-4 absolute
            assert np.allclose(got.reshape(batch, feature)[1:].sum(axis=1), 1.0, atol=1e-5)
        else:
            got, want = orc.bf16_to_f32(ws.read(1, xin.nbytes, np.uint16)), orc.bf16_to_f32(want)
            assert norm_max_err(got, want) <= 1e-2 and np.mean(got.view(np.uint32) == want.view(np.uint32)) > 0.98


def test_layer_norm_rows(backend):
    # layer_norm_float (cpu/float_kernels.rs:1338-1445); parallel sums differ from the CPU's left-to-right
    # sums by rounding only; absent gamma / beta are the identity affine
    for batch, feature, dt, affine in ((16, 256, kc.DTYPE_F32, True), (8, 33, kc.DTYPE_F32, False), (64, 4096, BF, True)):
        rng = np.random.default_rng(feature + batch)
        x, g, bt = (rng.standard_normal(n).astype(np.float32) for n in (batch * feature, feature, feature))
        if dt != kc.DTYPE_F32:
            x, g, bt = (orc.f32_to_bf16_rne(v) for v in (x, g, bt))
        ws = hb.DeviceWorkspace(backend, 4)
        ws.put(0, x)
        ws.put(1, g)
        ws.put(2, bt)
        ws.alloc(3, x.nbytes)
        call = kc.NormCall(kc.rb(0), kc.rb(1) if affine else kc.NONE, kc.rb(2) if affine else kc.NONE, kc.NONE, kc.rb(3),
                           batch, feature, 0, 0, f32bits(1e-5), dt)
        backend.dispatch(kc.KernelCall.LayerNorm(call), ws)
        want = orc.layer_norm(x, g if affine else None, bt if affine else None, batch, feature, f32bits(1e-5), dt)
        if dt == kc.DTYPE_F32:
            assert np.allclose(ws.read(3, x.nbytes, np.float32), want, rtol=1e-4, atol=2e-6)
        else:
            got, want = orc.bf16_to_f32(ws.read(3, x.nbytes, np.uint16)), orc.bf16_to_f32(want)
            assert norm_max_err(got, want) <= 1e-2 and np.mean(got.view(np.uint32) == want.view(np.uint32)) > 0.97
    bad = kc.NormCall(kc.rb(0), kc.NONE, kc.NONE, kc.NONE, kc.rb(3), 1, 8, 0, 0, f32bits(-1e-5), kc.DTYPE_F32)
    with pytest.raises(hb.BackendError):
        backend.dispatch(kc.KernelCall.LayerNorm(bad), ws)


def test_expand_and_broadcast_binary(backend):
    # expand_float / broadcast_binary_float (cpu/float_kernels.rs:3405-3444, :3250-3397): bit-exact
    rng = np.random.default_rng(72)
    for in_dims, out_dims in (((1, 5, 1, 7), (3, 5, 4, 7)), ((6, 1), (6, 33)), ((1,), (19,)), ((2, 1, 4096), (2, 3, 4096))):
        nin, nout = int(np.prod(in_dims)), int(np.prod(out_dims))
        for dt, store in ((kc.DTYPE_F32, np.float32), (BF, np.uint16)):
            small = rng.standard_normal(nin).astype(np.float32)
            other = rng.standard_normal(nout).astype(np.float32)
            if dt == BF:
                small, other = orc.f32_to_bf16_rne(small), orc.f32_to_bf16_rne(other)
            es = small.itemsize
            ws = hb.DeviceWorkspace(backend, 3)
            ws.put(0, small)
            ws.put(1, other)
            ws.alloc(2, nout * es)
            backend.dispatch(kc.KernelCall.Expand(kc.ExpandCall.make(kc.rb(0), kc.rb(2), in_dims, out_dims, dt)), ws)
            want = orc.broadcast(small, None, in_dims, out_dims, es)
            assert np.array_equal(ws.read(2, nout * es, np.uint8), want)
            assert np.array_equal(want.view(store).reshape(out_dims), np.broadcast_to(small.reshape(in_dims), out_dims))
            for op in (kc.BROADCAST_ADD, kc.BROADCAST_SUB, kc.BROADCAST_MUL):
                for lhs in (True, False):
                    call = kc.BroadcastBinaryCall.make(kc.rb(0), kc.rb(1), kc.rb(2), in_dims, out_dims, op, lhs, dt)
                    backend.dispatch(kc.KernelCall.BroadcastBinary(call), ws)
                    want = orc.broadcast(small, other, in_dims, out_dims, es, op, lhs, dt)
                    assert np.array_equal(ws.read(2, nout * es, np.uint8), want)
            ws.close()
    ws = hb.DeviceWorkspace(backend, 3)
    for i in range(3):
        ws.alloc(i, 1024)
    with pytest.raises(hb.BackendError) as e:   # an axis that is neither 1 nor equal cannot broadcast
        backend.dispatch(kc.KernelCall.Expand(kc.ExpandCall.make(kc.rb(0), kc.rb(2), (2, 3), (2, 6), BF)), ws)
    assert e.value.variant == "UnsupportedOp"
    with pytest.raises(hb.BackendError):
        backend.dispatch(kc.KernelCall.BroadcastBinary(kc.BroadcastBinaryCall.make(kc.rb(0), kc.rb(1), kc.rb(2), (1, 3), (2, 3), 7, True, BF)), ws)


def test_reduce_variants(backend):
    # reduce_float (cpu/float_kernels.rs:1901-2022): each cell folds in linear input order -> bit-exact, also with
    # the per-step narrowing of a 16-bit dtype; only the f32 full sum is order-relaxed (on the CPU too)
    rng = np.random.default_rng(59)
    ctors = ((kc.KernelCall.ReduceSum, 0, False), (kc.KernelCall.ReduceMean, 0, True), (kc.KernelCall.ReduceProd, 1, False),
             (kc.KernelCall.ReduceMin, 2, False), (kc.KernelCall.ReduceMax, 3, False))
    for dims, mask in (((64, 4096), 0b10), ((3, 4, 5, 2), 0b1010), ((7, 33, 5), 0b001), ((6, 50), 0b01), ((1000,), 0), ((4, 9), 0b11)):
        n = int(np.prod(dims))
        for dt in (kc.DTYPE_F32, BF):
            x = (rng.standard_normal(n) * 0.7 + 1.0).astype(np.float32)
            xin = x if dt == kc.DTYPE_F32 else orc.f32_to_bf16_rne(x)
            ws = hb.DeviceWorkspace(backend, 2)
            ws.put(0, xin)
            ws.alloc(1, xin.nbytes)
            for ctor, kind, mean in ctors:
                backend.dispatch(ctor(kc.ReduceCall.make(kc.rb(0), kc.rb(1), dims, mask, dt)), ws)
                want = orc.reduce(xin, dims, mask, kind, mean, dt)
                got = ws.read(1, want.nbytes, want.dtype)
                if dt == kc.DTYPE_F32 and want.size == 1 and kind == 0:
                    assert np.allclose(got, want, rtol=1e-5)
                else:
                    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (dims, mask, kind, dt)
            ws.close()
    ws = hb.DeviceWorkspace(backend, 2)
    ws.alloc(0, 1024)
    ws.alloc(1, 1024)
    bad = kc.ReduceCall.make(kc.rb(0), kc.rb(1), (4, 4), 0b01, BF)
    bad.element_count = 17
    with pytest.raises(hb.BackendError) as e:
        backend.dispatch(kc.KernelCall.ReduceSum(bad), ws)
    assert e.value.variant == "UnsupportedOp"


def test_exact_elementwise_variants(backend):
    # unary_float / binary_float with one IEEE operation per element (cpu/float_kernels.rs:190-296, :3446-3500,
    # :3660-3733): bit-exact, every 16-bit code for the unary forms (NaN inputs included)
    codes = np.arange(65536, dtype=np.uint16)
    rng = np.random.default_rng(45)
    special = np.array([0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, np.inf, -np.inf, 3e38, -3e38, 1e-40, -1e-40], dtype=np.float32)
    f32 = np.concatenate([special, (rng.standard_normal(4096 - special.size) * 7).astype(np.float32)])
    for tag in kc.EXACT_UNARY:
        for dt, x in ((BF, codes), (kc.DTYPE_F16, codes), (kc.DTYPE_F32, f32)):
            ws = hb.DeviceWorkspace(backend, 2)
            ws.put(0, x)
            ws.alloc(1, x.nbytes)
            backend.dispatch(kc.KernelCall.Elementwise(tag, kc.UnaryCall(kc.rb(0), kc.rb(1), x.size, 0, dt)), ws)
            want = orc.elementwise(tag, x, None, dt)
            got = ws.read(1, x.nbytes, x.dtype)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (tag, dt, np.flatnonzero(got.view(np.uint8) != want.view(np.uint8))[:4])
            ws.close()
    a32 = np.concatenate([np.repeat(special, special.size), (rng.standard_normal(4096) * 5).astype(np.float32)])
    b32 = np.concatenate([np.tile(special, special.size), (rng.standard_normal(4096) * 3).astype(np.float32)])
    for tag in kc.EXACT_BINARY:
        for dt in (kc.DTYPE_F32, BF, kc.DTYPE_F16):
            a, b = (a32, b32) if dt == kc.DTYPE_F32 else ((orc.f32_to_bf16_rne(a32), orc.f32_to_bf16_rne(b32)) if dt == BF else
                                                           (a32.astype(np.float16).view(np.uint16), b32.astype(np.float16).view(np.uint16)))
            ws = hb.DeviceWorkspace(backend, 3)
            ws.put(0, a)
            ws.put(1, b)
            ws.alloc(2, a.nbytes)
            backend.dispatch(kc.KernelCall.Elementwise(tag, kc.BinaryCall(kc.rb(0), kc.rb(1), kc.rb(2), a.size, 0, dt)), ws)
            want = orc.elementwise(tag, a, b, dt)
            got = ws.read(2, a.nbytes, a.dtype)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (tag, dt, np.flatnonzero(got.view(np.uint8) != want.view(np.uint8))[:4])
            ws.close()


def test_dequant_activation_table(backend):
    # dequant_activation (cpu/kernels.rs:311-381): bit-exact; every code, odd lengths, unaligned input, i4 nibbles
    rng = np.random.default_rng(113)
    for qd, act, n, off in ((kc.DTYPE_I8, kc.LUT_GELU, 256, 0), (kc.DTYPE_I8, kc.LUT_SILU, 1 << 20, 0), (kc.DTYPE_U8, kc.LUT_TANH, 100003, 0),
                            (kc.DTYPE_I8, kc.LUT_SIGMOID, 5000, 3), (kc.DTYPE_I4, kc.LUT_GELU, 4097, 0)):
        nbytes = (n + 1) // 2 if qd == kc.DTYPE_I4 else n
        codes = np.arange(256, dtype=np.uint8) if n == 256 else rng.integers(0, 256, size=nbytes, dtype=np.uint8)
        scale, zp = np.float32(0.05), -7
        ws = hb.DeviceWorkspace(backend, 2)
        ws.put(0, np.concatenate([np.zeros(off, np.uint8), codes]))
        ws.alloc(1, n * 4)
        call = kc.DequantActivationCall(kc.rb(0, off, nbytes), kc.rb(1), n, qd, act, kc.DTYPE_F32, int(scale.view(np.uint32)), zp)
        backend.dispatch(kc.KernelCall.DequantActivation(call), ws)
        want = orc.dequant_activation(codes, n, qd, act, scale, zp)
        assert np.array_equal(ws.read(1, n * 4, np.float32).view(np.uint32), want.view(np.uint32)), (qd, act, n)
        ws.close()


def test_where_selects_by_condition_bytes(backend):
    # where_float (cpu/float_kernels.rs:2908-2937): bit-exact, every 16-bit code on both sides
    rng = np.random.default_rng(78)
    codes = np.arange(65536, dtype=np.uint16)
    for dt, a, b in ((BF, codes, codes[::-1].copy()), (kc.DTYPE_F16, codes, codes[::-1].copy()),
                     (kc.DTYPE_F32, rng.standard_normal(5001).astype(np.float32), rng.standard_normal(5001).astype(np.float32))):
        cond = rng.integers(0, 3, size=a.size, dtype=np.uint8)      # 0 picks b, anything else a
        ws = hb.DeviceWorkspace(backend, 4)
        for i, v in enumerate((cond, a, b)):
            ws.put(i, v)
        ws.alloc(3, a.nbytes)
        backend.dispatch(kc.KernelCall.Where(kc.WhereCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), a.size, dt)), ws)
        want = orc.where(cond, a, b, dt)
        assert np.array_equal(ws.read(3, a.nbytes, a.dtype).view(np.uint8), want.view(np.uint8))
        ws.close()
