"""Decode attention on the GPU against the oracle composition (through the C ABI).

Parity definition for the int8-KV form: out = Cast(DecodeAttentionValid_f32(Cast(q),
Dequantize(K), Dequantize(V), ...)). Tolerance: max|err| / max|ref| <= 1e-2 for bf16 output
(the reference's own bf16 attention bound is 3e-2, crates/hologram-compute/tests/conformance.rs:1390);
<= 2e-4 when q/out are f32 (isolates the kernel's own arithmetic from the final bf16 truncation).
"""
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc
from helpers import norm_max_err, synth_bf16

pytestmark = pytest.mark.gpu
BF, F32 = kc.DTYPE_BF16, kc.DTYPE_F32


def make_q8_case(b, h, kv, past, d, seed, dtype=BF, m=1, sigma=1.0):
    rng = np.random.default_rng(seed)
    if dtype == BF:
        q = synth_bf16(b * h * m * d, 1.0, seed + 1)
    else:
        q = rng.standard_normal(b * h * m * d).astype(np.float32)
    src = {}
    for off, (name, rows) in enumerate((("kp", b * kv * past), ("vp", b * kv * past), ("kn", b * kv * m), ("vn", b * kv * m))):
        x = synth_bf16(rows * d, sigma, seed + 101 * (off + 2))
        src[name] = x
    quant = {k: orc.quantize_rows_i8(v, BF, v.size // d, d) for k, v in src.items()}
    return q, src, quant


def run_q8(backend, q, quant, valid_len, b, h, kv, m, past, d, dtype, scale_bits=0):
    ws = hb.DeviceWorkspace(backend, 12)
    ws.put(0, q)
    slot = 1
    for name in ("kp", "vp", "kn", "vn"):
        codes, scales = quant[name]
        ws.put(slot, codes if codes.size else np.zeros(16, np.int8))
        ws.put(slot + 1, scales if scales.size else np.zeros(4, np.float32))
        slot += 2
    ws.put(9, np.array([valid_len], dtype=np.uint32))
    es = 2 if dtype != F32 else 4
    ws.alloc(10, b * h * m * d * es)
    call = kc.DecodeAttentionValidQ8Call(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(6), kc.rb(7),
                                         kc.rb(8), kc.rb(9), kc.rb(10), b, h, kv, m, past, m, d, scale_bits, dtype)
    backend.dispatch(kc.KernelCall.DecodeAttentionValidQ8(call), ws)
    out = ws.read(10, b * h * m * d * es, np.uint16 if dtype != F32 else np.float32)
    ws.close()
    return out


def oracle_q8(q, quant, valid_len, b, h, kv, m, past, d, dtype, scale_bits=0):
    rc, out = orc.decode_attention_valid_q8(q, dtype, quant["kp"][0], quant["kp"][1], quant["vp"][0], quant["vp"][1],
                                            quant["kn"][0], quant["kn"][1], quant["vn"][0], quant["vn"][1], valid_len,
                                            b, h, kv, m, past, m, d, scale_bits)
    assert rc == 0
    return out


def as_f32(x, dtype):
    return x if dtype == F32 else orc.bf16_to_f32(x)


@pytest.mark.parametrize("b,h,kv,past,valid,dtype,tol", [
    (2, 32, 8, 1024, 1024, BF, 1e-2),
    (2, 32, 8, 1024, 1024, F32, 2e-4),
    (3, 8, 2, 1156, 700, BF, 1e-2),       # ragged valid_len inside a tile, past not a tile multiple
    (3, 8, 2, 1156, 700, F32, 2e-4),
    (1, 4, 4, 512, 512, F32, 2e-4),       # multi-head (group 1)
    (2, 8, 4, 384, 100, F32, 2e-4),       # group 2
    (1, 4, 1, 12, 12, F32, 2e-4),         # bucket smaller than a tile
    (1, 4, 1, 4096, 5, F32, 2e-4),        # realized prefix far below the bucket
    (2, 16, 2, 256, 256, F32, 2e-4),      # group 8: served by the general-shape kernel
    (1, 4, 2, 130, 130, F32, 2e-4),       # bucket not a multiple of 4: general-shape kernel
])
def test_q8_attention_matches_oracle(backend, b, h, kv, past, valid, dtype, tol):
    d = 128
    q, _, quant = make_q8_case(b, h, kv, past, d, seed=past + h, dtype=dtype)
    got = run_q8(backend, q, quant, valid, b, h, kv, 1, past, d, dtype)
    want = oracle_q8(q, quant, valid, b, h, kv, 1, past, d, dtype)
    assert norm_max_err(as_f32(got, dtype), as_f32(want, dtype)) <= tol


def test_q8_unrealized_rows_are_never_read(backend):
    # padded == tight (tests/decode_attention_valid.rs:226-282): bytes beyond valid_len do not matter
    b, h, kv, past, d, valid = 2, 8, 2, 512, 128, 300
    q, _, quant = make_q8_case(b, h, kv, past, d, seed=77, dtype=F32)
    a = run_q8(backend, q, quant, valid, b, h, kv, 1, past, d, F32)
    rng = np.random.default_rng(1)
    dirty = dict(quant)
    for name in ("kp", "vp"):
        codes, scales = (v.copy() for v in quant[name])
        c3 = codes.reshape(b * kv, past, d)
        c3[:, valid:, :] = rng.integers(-128, 128, size=c3[:, valid:, :].shape)
        s2 = scales.reshape(b * kv, past)
        s2[:, valid:] = np.float32(np.nan)
        dirty[name] = (codes, scales)
    bdirty = run_q8(backend, q, dirty, valid, b, h, kv, 1, past, d, F32)
    assert np.array_equal(a.view(np.uint32), bdirty.view(np.uint32))
    # valid_len beyond the bucket means the whole bucket
    full = run_q8(backend, q, quant, past, b, h, kv, 1, past, d, F32)
    over = run_q8(backend, q, quant, 10 ** 9, b, h, kv, 1, past, d, F32)
    assert np.array_equal(full.view(np.uint32), over.view(np.uint32))


def test_q8_extreme_rows(backend):
    # a zero query head, zero-scale (all-zero) K/V rows, one huge V row, a dominant key
    b, h, kv, past, d = 1, 4, 1, 640, 128
    q, src, _ = make_q8_case(b, h, kv, past, d, seed=5, dtype=F32)
    q = q.reshape(h, d)
    q[1] = 0.0
    q[2] *= 40.0          # very peaked softmax
    q[3] *= 1e-3
    q = q.reshape(-1)
    kp = orc.bf16_to_f32(src["kp"]).reshape(past, d)
    vp = orc.bf16_to_f32(src["vp"]).reshape(past, d)
    kp[10] = 0.0
    vp[11] = 0.0
    vp[500] *= 3e4
    kp[600] *= 30.0
    src["kp"], src["vp"] = orc.f32_to_bf16_rne(kp.reshape(-1)), orc.f32_to_bf16_rne(vp.reshape(-1))
    quant = {k: orc.quantize_rows_i8(v, BF, v.size // d, d) for k, v in src.items()}
    got = run_q8(backend, q, quant, past, b, h, kv, 1, past, d, F32)
    want = oracle_q8(q, quant, past, b, h, kv, 1, past, d, F32)
    got, want = got.reshape(h, d), want.reshape(h, d)
    for head in range(h):
        assert norm_max_err(got[head], want[head]) <= 5e-4, head


def test_q8_explicit_scale_and_general_kernel_shapes(backend):
    import struct
    sb = struct.unpack("<I", struct.pack("<f", 0.05))[0]
    for (b, h, kv, m, past, d) in [(2, 8, 2, 1, 256, 128), (1, 6, 3, 4, 40, 64), (1, 2, 2, 3, 0, 32)]:
        q, _, quant = make_q8_case(b, h, kv, past, d, seed=d + m, dtype=F32, m=m)
        got = run_q8(backend, q, quant, past, b, h, kv, m, past, d, F32, scale_bits=sb)
        want = oracle_q8(q, quant, past, b, h, kv, m, past, d, F32, scale_bits=sb)
        assert norm_max_err(got, want) <= 2e-4


def test_unquantized_decode_attention_valid(backend):
    # the reference variant itself (KernelCall::DecodeAttentionValid, wire 121) in bf16 and f32
    b, h, kv, m, past, d = 1, 4, 2, 4, 12, 16
    for dtype, tol in ((F32, 1e-5), (BF, 3e-2)):
        rng = np.random.default_rng(3)
        arrs = [rng.standard_normal(n).astype(np.float32) for n in
                (b * h * m * d, b * kv * past * d, b * kv * past * d, b * kv * m * d, b * kv * m * d)]
        if dtype == BF:
            arrs = [orc.f32_to_bf16_rne(a) for a in arrs]
        for valid in (0, 5, 12, 99):
            ws = hb.DeviceWorkspace(backend, 7)
            for i, a in enumerate(arrs):
                ws.put(i, a)
            ws.put(5, np.array([valid], dtype=np.uint32))
            ws.alloc(6, arrs[0].nbytes)
            call = kc.DecodeAttentionValidCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(6),
                                               b, h, kv, m, past, m, d, 0, dtype)
            backend.dispatch(kc.KernelCall.DecodeAttentionValid(call), ws)
            got = ws.read(6, arrs[0].nbytes, np.float32 if dtype == F32 else np.uint16)
            rc, want = orc.decode_attention_valid(*arrs, valid, b, h, kv, m, past, m, d, 0, dtype)
            assert rc == 0
            assert norm_max_err(as_f32(got, dtype), as_f32(want, dtype)) <= tol
    # geometry refusals (float_kernels.rs:4205-4220)
    ws = hb.DeviceWorkspace(backend, 7)
    for i in range(7):
        ws.alloc(i, 4096)
    for bad in (kc.DecodeAttentionValidCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(6), 1, 4, 2, 2, 4, 1, 16, 0, F32),
                kc.DecodeAttentionValidCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(6), 1, 4, 3, 1, 4, 1, 16, 0, F32)):
        with pytest.raises(hb.BackendError) as e:
            backend.dispatch(kc.KernelCall.DecodeAttentionValid(bad), ws)
        assert e.value.variant == "UnsupportedOp"


def test_mask_form_decode_attention(backend):
    # KernelCall::DecodeAttention (wire 119): additive f32 mask [q_rows, past + new], every key takes
    # part, -inf erases exactly, an all-erased row is the zero vector, q_rows independent of new_len
    b, h, kv, m, past, new, d = 2, 4, 2, 3, 37, 2, 32
    l = past + new
    for dtype, tol in ((F32, 1e-5), (BF, 3e-2)):
        rng = np.random.default_rng(8)
        arrs = [rng.standard_normal(n).astype(np.float32) for n in
                (b * h * m * d, b * kv * past * d, b * kv * past * d, b * kv * new * d, b * kv * new * d)]
        if dtype == BF:
            arrs = [orc.f32_to_bf16_rne(a) for a in arrs]
        mask = np.where(rng.random((m, l)) < 0.3, -np.inf, 0.0).astype(np.float32)
        mask[0, 5] = 0.75            # a finite bias
        mask[1, :] = -np.inf         # every key erased: zero vector
        for scale_bits in (0, int(np.float32(0.2).view(np.uint32))):
            ws = hb.DeviceWorkspace(backend, 7)
            for i, a in enumerate(arrs):
                ws.put(i, a)
            ws.put(5, mask)
            ws.alloc(6, arrs[0].nbytes)
            call = kc.DecodeAttentionCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(6),
                                          b, h, kv, m, past, new, d, scale_bits, dtype)
            backend.dispatch(kc.KernelCall.DecodeAttention(call), ws)
            got = as_f32(ws.read(6, arrs[0].nbytes, np.float32 if dtype == F32 else np.uint16), dtype)
            want = as_f32(orc.decode_attention_mask(*arrs, mask, b, h, kv, m, past, new, d, scale_bits, dtype), dtype)
            assert norm_max_err(got, want) <= tol
            assert not np.any(got.reshape(b * h, m, d)[:, 1, :])
    # the realized-length mask reproduces the scalar form (decode step: m = new = 1)
    b, h, kv, past, d, valid = 1, 4, 2, 24, 16, 9
    rng = np.random.default_rng(4)
    arrs = [rng.standard_normal(n).astype(np.float32) for n in (b * h * d, b * kv * past * d, b * kv * past * d, b * kv * d, b * kv * d)]
    mask = np.zeros((1, past + 1), np.float32)
    mask[0, valid:past] = -np.inf
    ws = hb.DeviceWorkspace(backend, 9)
    for i, a in enumerate(arrs):
        ws.put(i, a)
    ws.put(5, mask)
    ws.put(6, np.array([valid], dtype=np.uint32))
    ws.alloc(7, arrs[0].nbytes)
    ws.alloc(8, arrs[0].nbytes)
    backend.dispatch(kc.KernelCall.DecodeAttention(kc.DecodeAttentionCall(
        kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(7), b, h, kv, 1, past, 1, d, 0, F32)), ws)
    backend.dispatch(kc.KernelCall.DecodeAttentionValid(kc.DecodeAttentionValidCall(
        kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(6), kc.rb(8), b, h, kv, 1, past, 1, d, 0, F32)), ws)
    assert norm_max_err(ws.read(7, arrs[0].nbytes, np.float32), ws.read(8, arrs[0].nbytes, np.float32)) <= 1e-6
    # refusals: no key at all; heads not a multiple of kv_heads
    for bad in (kc.DecodeAttentionCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(7), 1, 4, 2, 1, 0, 0, 16, 0, F32),
                kc.DecodeAttentionCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(7), 1, 4, 3, 1, 4, 1, 16, 0, F32)):
        with pytest.raises(hb.BackendError) as e:
            backend.dispatch(kc.KernelCall.DecodeAttention(bad), ws)
        assert e.value.variant == "UnsupportedOp"


def test_config4_full_size_codes_and_attention(backend):
    # batch 32, 32 query / 8 kv heads, head_dim 128, 8192 cached positions: quantizer codes
    # bit-exact on the full cache, attention within tolerance of the oracle on every row.
    b, h, kv, past, d = 32, 32, 8, 8192, 128
    rows = b * kv * past
    q = synth_bf16(b * h * d, 1.0, 0xC4)
    ws = hb.DeviceWorkspace(backend, 12)
    ws.put(0, q)
    quant = {}
    slot = 1
    for name, nrows, seed in (("kp", rows, 1), ("vp", rows, 2), ("kn", b * kv, 3), ("vn", b * kv, 4)):
        src = synth_bf16(nrows * d, 1.0, 0xC4 + seed)
        quant[name] = orc.quantize_rows_i8(src, BF, nrows, d)
        tmp = hb.DeviceWorkspace(backend, 1)
        tmp.put(0, src)
        ptr, nbytes = tmp.slot(0)
        ws.alloc(slot, nrows * d)
        ws.alloc(slot + 1, nrows * 4)
        stage = hb.DeviceWorkspace(backend, 3)
        stage.bind(0, ptr, nbytes)
        for j in (0, 1):
            p, nb = ws.slot(slot + j)
            stage.bind(1 + j, p, nb)
        backend.dispatch(kc.KernelCall.QuantizeRowsI8(kc.QuantizeRowsI8Call(kc.rb(0), kc.rb(1), kc.rb(2), nrows, d, BF)), stage)
        backend.synchronize()
        assert np.array_equal(ws.read(slot, nrows * d, np.int8), quant[name][0]), name
        assert np.array_equal(ws.read(slot + 1, nrows * 4, np.uint32), quant[name][1].view(np.uint32)), name
        tmp.close()
        slot += 2
    ws.put(9, np.array([past], dtype=np.uint32))
    ws.alloc(10, b * h * d * 2)
    call = kc.DecodeAttentionValidQ8Call(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), kc.rb(5), kc.rb(6), kc.rb(7),
                                         kc.rb(8), kc.rb(9), kc.rb(10), b, h, kv, 1, past, 1, d, 0, BF)
    backend.dispatch(kc.KernelCall.DecodeAttentionValidQ8(call), ws)
    got = orc.bf16_to_f32(ws.read(10, b * h * d * 2, np.uint16))
    want = orc.bf16_to_f32(oracle_q8(q, quant, past, b, h, kv, 1, past, d, BF))
    err = norm_max_err(got, want)
    print(f"config-4 attention: max|err|/max|ref| = {err:.3e}")
    assert err <= 1e-2


def test_legacy_attention_prefill_form(backend):
    # KernelCall::Attention (wire 69; attention_float, cpu/float_kernels.rs:2244-2395): the reference's own
    # conformance cases plus a longer bf16 prefill; online softmax on the GPU against the CPU's two-pass row
    from helpers import ATTENTION_CASES
    cases = [(c, kc.DTYPE_F32) for c in ATTENTION_CASES] + [((2, 8, 2, 160, 128, True, None), BF), ((1, 4, 4, 96, 64, False, None), BF)]
    for idx, ((b, h, hkv, s, d, causal, mult), dt) in enumerate(cases):
        rng = np.random.default_rng(0x8c0 + idx)
        q, k, v = (rng.standard_normal(n).astype(np.float32) for n in (b * h * s * d, b * hkv * s * d, b * hkv * s * d))
        if dt == BF:
            q, k, v = (orc.f32_to_bf16_rne(x) for x in (q, k, v))
        bits = int(np.float32(mult).view(np.uint32)) if mult else 0
        kvh = hkv if hkv != h else 0
        ws = hb.DeviceWorkspace(backend, 4)
        for i, x in enumerate((q, k, v)):
            ws.put(i, x)
        ws.alloc(3, q.nbytes)
        call = kc.AttentionCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), b, h, s, d, kvh, int(causal), bits, dt)
        backend.dispatch(kc.KernelCall.Attention(call), ws)
        want = orc.attention(q, k, v, b, h, kvh, s, d, causal, bits, dt)
        got = ws.read(3, q.nbytes, q.dtype)
        if dt == BF:
            got, want = orc.bf16_to_f32(got), orc.bf16_to_f32(want)
        assert norm_max_err(got, want) <= (1e-2 if dt == BF else 2e-4), (idx, norm_max_err(got, want))
        ws.close()
