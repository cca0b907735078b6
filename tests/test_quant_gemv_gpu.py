"""Output-major W8A8 decode product (KernelCall::MatMulDequant, wire 116) on the GPU: exact-integer
arithmetic, so every output bit must equal the CPU kernel's, including the reference's own FNV-1a-64
golden (crates/hologram-compute/src/cpu/simd.rs:8236-8262)."""
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
F32, I8 = kc.DTYPE_F32, kc.DTYPE_I8


def run(backend, a, bq, scales, m, k, n, residual=None, act=0, zero_points=None, quant=I8, codebook=None):
    ws = hb.DeviceWorkspace(backend, 7)
    ws.put(0, a)
    ws.put(1, bq)
    ws.put(2, scales)
    ws.put(3, np.zeros(n, dtype=np.int32) if zero_points is None else zero_points)
    ws.alloc(4, m * n * 4)
    res = kc.NONE
    if residual is not None:
        ws.put(5, residual)
        res = kc.rb(5)
    call = kc.MatMulDequantCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), m, k, n, n, 1, quant, F32, 0, 0, 1, 1, act, res)
    if codebook is not None:
        ws.put(6, codebook)
        call.codebook = kc.rb(6)
    backend.dispatch(kc.KernelCall.MatMulDequant(call), ws)
    out = ws.read(4, m * n * 4, np.float32).copy()
    ws.close()
    return out


def test_reference_golden_fixture(backend):
    m, k, n = 3, 64, 24
    a = (np.array([float(i * 37 % 91) for i in range(m * k)], dtype=np.float32) - np.float32(45.0)) * np.float32(0.031)
    scales = np.float32(0.011) + np.arange(n, dtype=np.float32) * np.float32(0.0007)
    bq = np.array([(i * 31 % 255) - 127 for i in range(k * n)], dtype=np.int8)
    out = run(backend, a, bq, scales, m, k, n)
    assert orc.fnv1a64_f32(out) == 0x787CCDC172029F9B


@pytest.mark.parametrize("m,k,n", [(1, 4096, 14336), (4, 896, 4864), (1, 100, 7), (9, 250, 33), (2, 4096, 4096),
                                   (3, 14336, 130), (8, 1024, 1001), (9, 512, 37), (5, 16384, 21), (2, 16400, 9), (1, 64, 3)])
def test_bit_exact_against_the_cpu_kernel(backend, m, k, n):
    rng = np.random.default_rng(m * 7 + n)
    a = rng.standard_normal(m * k).astype(np.float32)
    if m > 1:
        a[:k] = 0.0                                   # a zero activation row gives a zero output row
    bq = rng.integers(-127, 128, size=n * k, dtype=np.int8)
    scales = (rng.random(n).astype(np.float32) + np.float32(0.01)) * np.float32(0.02)
    got = run(backend, a, bq, scales, m, k, n)
    want = orc.matmul_w8a8_omajor(a, bq, scales, m, k, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    if m > 1:
        assert not got[:n].any()


def test_epilogue_and_refusals(backend):
    m, k, n = 2, 512, 96
    rng = np.random.default_rng(3)
    a = rng.standard_normal(m * k).astype(np.float32)
    bq = rng.integers(-127, 128, size=n * k, dtype=np.int8)
    scales = (rng.random(n).astype(np.float32) + np.float32(0.01)) * np.float32(0.01)
    r = rng.standard_normal(m * n).astype(np.float32)
    got = run(backend, a, bq, scales, m, k, n, residual=r, act=kc.FUSED_SILU)
    want = orc.matmul_w8a8_omajor(a, bq, scales, m, k, n, residual=r, act=kc.LUT_SILU)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # contract violations fail loud (cpu/float_kernels.rs:546-566)
    ws = hb.DeviceWorkspace(backend, 5)
    for i in range(5):
        ws.alloc(i, 1 << 16)
    base = [kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), 1, 64, 16, 16, 1, I8, F32, 0, 0]
    for tail in ([1, 0, 0, kc.NONE], [0, 1, 0, kc.NONE]):          # unpaired omajor / W8A8 (the [k,n] form with f32 activations is served)
        with pytest.raises(hb.BackendError) as e:
            backend.dispatch(kc.KernelCall.MatMulDequant(kc.MatMulDequantCall(*base, *tail)), ws)
        assert e.value.variant == "UnsupportedOp"
    bad = list(base)
    bad[8] = 8                                                                          # channels != n
    with pytest.raises(hb.BackendError) as e:
        backend.dispatch(kc.KernelCall.MatMulDequant(kc.MatMulDequantCall(*bad, 1, 1, 0, kc.NONE)), ws)
    assert e.value.variant == "UnsupportedOp"
    # a non-zero zero point is not the symmetric form: reported at the next synchronising call
    zp = np.zeros(n, dtype=np.int32)
    zp[5] = 3
    with pytest.raises(hb.BackendError):
        run(backend, a, bq, scales, m, k, n, zero_points=zp)


def test_packed_i4_reference_golden_and_bit_exactness(backend):
    # W4A8: [n, k/2] packed signed nibbles, low nibble first (matmul_i4_pc_omajor, cpu/simd.rs:6164-6260); the
    # reference's FNV golden for this tier (:8257-8265), then seeded shapes against the CPU kernel
    m, k, n = 3, 64, 24
    a = (np.array([float(i * 37 % 91) for i in range(m * k)], dtype=np.float32) - np.float32(45.0)) * np.float32(0.031)
    scales = np.float32(0.011) + np.arange(n, dtype=np.float32) * np.float32(0.0007)
    bq4 = np.array([(i * 53 + 9) % 251 for i in range(k * n // 2)], dtype=np.uint8)
    assert orc.fnv1a64_f32(run(backend, a, bq4, scales, m, k, n, quant=kc.DTYPE_I4)) == 0x4C5123C024AF97AE
    for m, k, n in ((1, 4096, 14336), (4, 4096, 1001), (2, 14336, 130), (8, 1024, 77), (9, 512, 37), (1, 32768, 5), (3, 32, 3)):
        rng = np.random.default_rng(m * 11 + n)
        a = rng.standard_normal(m * k).astype(np.float32)
        if m > 1:
            a[:k] = 0.0
        bq = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)
        scales = (rng.random(n).astype(np.float32) + np.float32(0.01)) * np.float32(0.02)
        got = run(backend, a, bq, scales, m, k, n, quant=kc.DTYPE_I4)
        want = orc.matmul_w8a8_omajor(a, bq, scales, m, k, n, i4=True)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (m, k, n)
    with pytest.raises(hb.BackendError) as e:      # k = 48: columns of 24 bytes do not stream in 16-byte units
        run(backend, np.ones(48, np.float32), np.zeros(48, np.uint8), np.ones(2, np.float32), 1, 48, 2, quant=kc.DTYPE_I4)
    assert e.value.variant == "UnsupportedOp"


def test_e8_codebook_reference_golden_and_bit_exactness(backend):
    # W1A8: [n, k/8] indices into the model's 256 x 8 i8 codebook (matmul_e8cb_omajor, cpu/simd.rs:6845-6960; wire
    # form 117 with the codebook operand); the reference's FNV golden for this tier (:8266-8280), then seeded shapes
    m, k, n = 3, 64, 24
    a = (np.array([float(i * 37 % 91) for i in range(m * k)], dtype=np.float32) - np.float32(45.0)) * np.float32(0.031)
    scales = np.float32(0.011) + np.arange(n, dtype=np.float32) * np.float32(0.0007)
    cb = np.array([(i * 37 + 11) % 255 - 127 for i in range(256 * 8)], dtype=np.int8)
    bq8 = np.array([(i * 17 + 3) % 256 for i in range(n * (k // 8))], dtype=np.uint8)
    assert orc.fnv1a64_f32(run(backend, a, bq8, scales, m, k, n, quant=kc.DTYPE_E8CB, codebook=cb)) == 0x88AC55A91DD5AA0D
    rng = np.random.default_rng(117)
    cb = rng.integers(-127, 128, size=2048, dtype=np.int8)
    for m, k, n in ((1, 4096, 14336), (4, 4096, 1001), (2, 14336, 130), (9, 520, 37), (1, 8, 3)):
        a = rng.standard_normal(m * k).astype(np.float32)
        if m > 1:
            a[:k] = 0.0
        bq = rng.integers(0, 256, size=n * k // 8, dtype=np.uint8)
        scales = (rng.random(n).astype(np.float32) + np.float32(0.01)) * np.float32(0.02)
        got = run(backend, a, bq, scales, m, k, n, quant=kc.DTYPE_E8CB, codebook=cb)
        want = orc.matmul_w8a8_omajor(a, bq, scales, m, k, n, codebook=cb)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (m, k, n)
    for kwargs in (dict(quant=kc.DTYPE_E8CB), dict(quant=I8, codebook=cb)):      # the tier and the codebook operand go together
        with pytest.raises(hb.BackendError) as e:
            run(backend, np.ones(64, np.float32), np.zeros(64, np.uint8), np.ones(2, np.float32), 1, 64, 2, **kwargs)
        assert e.value.variant == "UnsupportedOp"


def run_kn(backend, a, bq, m, k, n, quant, scales=None, zero_points=None, channels=0, inner=1, scale=1.0, zero_point=0, residual=None, act=0):
    """MatMulDequant over a [k, n] weight with f32 activations (wire 111, or 116 when an epilogue is bound)."""
    ws = hb.DeviceWorkspace(backend, 6)
    ws.put(0, a)
    ws.put(1, bq)
    sc, zp, res = kc.NONE, kc.NONE, kc.NONE
    if scales is not None:
        ws.put(2, scales)
        ws.put(3, zero_points)
        sc, zp = kc.rb(2), kc.rb(3)
    if residual is not None:
        ws.put(5, residual)
        res = kc.rb(5)
    ws.alloc(4, m * n * 4)
    sb = int(np.float32(scale).view(np.uint32))
    call = kc.MatMulDequantCall(kc.rb(0), kc.rb(1), sc, zp, kc.rb(4), m, k, n, channels, inner, quant, F32, sb, zero_point, 0, 0, act, res)
    backend.dispatch(kc.KernelCall.MatMulDequant(call), ws)
    out = ws.read(4, m * n * 4, np.float32).copy()
    ws.close()
    return out


LUT_OF_FUSED = {kc.FUSED_GELU: kc.LUT_GELU, kc.FUSED_SILU: kc.LUT_SILU, kc.FUSED_TANH: kc.LUT_TANH}


@pytest.mark.parametrize("m,k,n", [(1, 64, 48), (3, 17, 33), (5, 9, 16), (1, 2048, 64), (2, 4096, 1000), (4, 128, 24), (1, 4096, 14336)])
def test_kn_form_per_channel_i8_is_bit_exact(backend, m, k, n):
    # m <= 3 with every zero point 0 takes the integer-level chain with the scale applied once (cpu/simd.rs:3480-3570);
    # m > 3, or a nonzero zero point, dequantizes first (cpu/float_kernels.rs:640-731): different bits, the reference's choice
    rng = np.random.default_rng(m * 131 + n)
    a = rng.standard_normal(m * k).astype(np.float32)
    bq = rng.integers(-127, 128, size=k * n, dtype=np.int8)
    scales = (rng.random(n, dtype=np.float32) * np.float32(0.02) + np.float32(0.001)).astype(np.float32)
    for zps in (np.zeros(n, dtype=np.int32), rng.integers(-3, 4, size=n, dtype=np.int32)):
        got = run_kn(backend, a, bq, m, k, n, I8, scales, zps, channels=n, inner=1)
        want = orc.matmul_dequant_kn(a, bq, m, k, n, I8, scales, zps, channels=n, inner=1)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_kn_form_tiers_layouts_and_epilogue(backend):
    rng = np.random.default_rng(17)
    m, k, n = 3, 96, 40
    a = rng.standard_normal(m * k).astype(np.float32)
    res = rng.standard_normal(m * n).astype(np.float32)
    # per-tensor u8 with a zero point, and a fused residual + activation (wire 116 with bq_omajor = act_quant = 0)
    bq = rng.integers(0, 256, size=k * n, dtype=np.uint8)
    got = run_kn(backend, a, bq, m, k, n, kc.DTYPE_U8, scale=0.0123, zero_point=131, residual=res, act=kc.FUSED_SILU)
    want = orc.matmul_dequant_kn(a, bq, m, k, n, kc.DTYPE_U8, scale=0.0123, zero_point=131, residual=res, act=LUT_OF_FUSED[kc.FUSED_SILU])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # packed i4 (two nibbles per byte, low first, index kk * n + j), per-channel along k (channels = k, inner = n)
    bq4 = rng.integers(0, 256, size=k * n // 2, dtype=np.uint8)
    sc = (rng.random(k, dtype=np.float32) * np.float32(0.1) + np.float32(0.01)).astype(np.float32)
    zp = rng.integers(-2, 3, size=k, dtype=np.int32)
    got = run_kn(backend, a, bq4, m, k, n, kc.DTYPE_I4, sc, zp, channels=k, inner=n, act=kc.FUSED_TANH)
    want = orc.matmul_dequant_kn(a, bq4, m, k, n, kc.DTYPE_I4, sc, zp, channels=k, inner=n, act=LUT_OF_FUSED[kc.FUSED_TANH])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # an output-major weight must never be read with the [k, n] interpretation, and W8A8 has one emitter
    ws = hb.DeviceWorkspace(backend, 5)
    for i in range(5):
        ws.alloc(i, 1 << 16)
    for omajor, act_quant in ((1, 0), (0, 1)):
        call = kc.MatMulDequantCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), 1, 64, 16, 16, 1, I8, F32, 0, 0, omajor, act_quant, 0, kc.NONE)
        with pytest.raises(hb.BackendError) as e:
            backend.dispatch(kc.KernelCall.MatMulDequant(call), ws)
        assert e.value.variant == "UnsupportedOp" and "paired" in str(e.value)
    ws.close()
