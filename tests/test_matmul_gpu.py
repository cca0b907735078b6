"""bf16 matmul (+ fused epilogues) on the GPU against the oracle (through the C ABI).

Tolerance: max|err| / max|ref| <= 1e-2 against the oracle's ascending-k fused-multiply-add
chain truncated to bf16 (the reference's own bf16 bound vs f64 is 8e-3,
crates/hologram-compute/tests/conformance.rs:256). Shapes that take the per-cell kernel run
the reference's exact recurrence and must match bit for bit.
"""
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc
from helpers import norm_max_err

pytestmark = pytest.mark.gpu
BF = kc.DTYPE_BF16


def synth(m, k, n, seed):
    rng = np.random.default_rng(seed)
    s = np.float32(1.0 / np.sqrt(k))
    a = orc.f32_to_bf16_rne(rng.standard_normal(m * k, dtype=np.float32) * s)
    b = orc.f32_to_bf16_rne(rng.standard_normal(k * n, dtype=np.float32) * s)
    return a, b


def run(backend, a, b, m, k, n, act=0, residual=None):
    ws = hb.DeviceWorkspace(backend, 4)
    ws.put(0, a)
    ws.put(1, b)
    ws.alloc(2, m * n * 2 + 64)
    mm = kc.MatMulCall(kc.rb(0), kc.rb(1), kc.rb(2), m, k, n, BF, 0)
    if residual is not None:
        ws.put(3, residual)
        call = kc.KernelCall.MatMulAdd(kc.MatMulAddCall(mm, kc.rb(3)))
    elif act:
        call = kc.KernelCall.MatMulActivation(kc.MatMulActivationCall(mm, act))
    else:
        call = kc.KernelCall.MatMul(mm)
    backend.dispatch(call, ws)
    out = ws.read(kc.rb(2, 0, m * n * 2), m * n * 2, np.uint16)
    assert not ws.read(kc.rb(2, m * n * 2), 64).any()
    ws.close()
    return out


@pytest.mark.parametrize("m,k,n", [(3, 37, 16), (5, 64, 20), (1, 8, 8), (7, 33, 9)])
def test_small_and_odd_shapes_are_bit_exact(backend, m, k, n):
    a, b = synth(m, k, n, m + k + n)
    assert np.array_equal(run(backend, a, b, m, k, n), orc.matmul(a, b, m, k, n, BF))


@pytest.mark.parametrize("m,k,n", [
    (128, 64, 128), (128, 256, 256), (200, 192, 512), (64, 512, 1024), (16, 4096, 1024), (64, 4096, 4096),
    (256, 1000 * 8, 136), (129, 72, 8 * 33), (1024, 1024, 1024), (40, 2048, 512), (100, 4096, 256), (64, 14336, 4096),
])
def test_tensor_core_path_within_tolerance(backend, m, k, n):
    a, b = synth(m, k, n, m * 7 + n)
    got = orc.bf16_to_f32(run(backend, a, b, m, k, n))
    want = orc.bf16_to_f32(orc.matmul(a, b, m, k, n, BF))
    assert norm_max_err(got, want) <= 1e-2


def test_fused_epilogues(backend):
    m, k, n = 64, 1024, 2048
    a, b = synth(m, k, n, 21)
    r = orc.f32_to_bf16_rne(np.random.default_rng(22).standard_normal(m * n, dtype=np.float32))
    plain = run(backend, a, b, m, k, n)
    silu = run(backend, a, b, m, k, n, act=kc.FUSED_SILU)
    add = run(backend, a, b, m, k, n, residual=r)
    # the epilogue acts on the truncated product exactly as the unfused pair would
    assert np.array_equal(silu, orc.unary_lut(kc.LUT_SILU, BF, plain))
    assert np.array_equal(add, orc.binary(0, plain, r, BF))
    want = orc.bf16_to_f32(orc.matmul(a, b, m, k, n, BF, act=kc.FUSED_SILU))
    assert norm_max_err(orc.bf16_to_f32(silu), want) <= 1e-2
    # split-K route (few tiles): same identities
    m, k, n = 16, 4096, 512
    a, b = synth(m, k, n, 23)
    r = orc.f32_to_bf16_rne(np.random.default_rng(24).standard_normal(m * n, dtype=np.float32))
    plain = run(backend, a, b, m, k, n)
    assert np.array_equal(run(backend, a, b, m, k, n, act=kc.FUSED_GELU), orc.unary_lut(kc.LUT_GELU, BF, plain))
    assert np.array_equal(run(backend, a, b, m, k, n, residual=r), orc.binary(0, plain, r, BF))


def test_refusals(backend):
    ws = hb.DeviceWorkspace(backend, 3)
    for i in range(3):
        ws.alloc(i, 1 << 16)
    with pytest.raises(hb.BackendError) as e:
        backend.dispatch(kc.KernelCall.MatMul(kc.MatMulCall(kc.rb(0), kc.rb(1), kc.rb(2), 64, 64, 64, kc.DTYPE_F64, 0)), ws)
    assert e.value.variant == "UnsupportedOp"
    with pytest.raises(hb.BackendError) as e:   # A shorter than m*k
        backend.dispatch(kc.KernelCall.MatMul(kc.MatMulCall(kc.rb(0), kc.rb(1), kc.rb(2), 1024, 64, 8, BF, 0)), ws)
    assert e.value.variant == "SlotOutOfRange" and e.value.slot == 0
    # m == 0 is a no-op (float_kernels.rs:302-304)
    backend.dispatch(kc.KernelCall.MatMul(kc.MatMulCall(kc.rb(0), kc.rb(1), kc.rb(2), 0, 64, 64, BF, 0)), ws)


def test_config3_prefill_4096_cubed(backend):
    m = k = n = 4096
    a, b = synth(m, k, n, 0xC3)
    got = orc.bf16_to_f32(run(backend, a, b, m, k, n))
    want = orc.bf16_to_f32(orc.matmul(a, b, m, k, n, BF))
    err = norm_max_err(got, want)
    print(f"4096^3 matmul: max|err|/max|ref| = {err:.3e}")
    assert err <= 1e-2


def test_config3_decode_16x4096x14336(backend):
    m, k, n = 16, 4096, 14336
    a, b = synth(m, k, n, 0xC3 + 1)
    got = orc.bf16_to_f32(run(backend, a, b, m, k, n))
    want = orc.bf16_to_f32(orc.matmul(a, b, m, k, n, BF))
    err = norm_max_err(got, want)
    print(f"16x4096x14336 matmul: max|err|/max|ref| = {err:.3e}")
    assert err <= 1e-2


def run_dt(backend, a, b, m, k, n, dt, act=0, residual=None):
    es = 4 if dt == kc.DTYPE_F32 else 2
    ws = hb.DeviceWorkspace(backend, 4)
    ws.put(0, a)
    ws.put(1, b)
    ws.alloc(2, m * n * es)
    mm = kc.MatMulCall(kc.rb(0), kc.rb(1), kc.rb(2), m, k, n, dt, 0)
    if residual is not None:
        ws.put(3, residual)
        call = kc.KernelCall.MatMulAdd(kc.MatMulAddCall(mm, kc.rb(3)))
    elif act:
        call = kc.KernelCall.MatMulActivation(kc.MatMulActivationCall(mm, act))
    else:
        call = kc.KernelCall.MatMul(mm)
    backend.dispatch(call, ws)
    out = ws.read(2, m * n * es, np.float32 if dt == kc.DTYPE_F32 else np.uint16)
    ws.close()
    return out


def f16_to_f32(h):
    return h.view(np.float16).astype(np.float32)


@pytest.mark.parametrize("m,k,n", [(64, 1024, 2048), (16, 4096, 512), (200, 192, 512), (5, 64, 20)])
def test_f16_matmul(backend, m, k, n):
    # f16 takes the same tensor-core kernel (operand format f16, the reference's add-half narrow);
    # the last shape takes the per-cell kernel and is bit-exact
    rng = np.random.default_rng(m + n)
    s = np.float32(1.0 / np.sqrt(k))
    a = (rng.standard_normal(m * k, dtype=np.float32) * s).astype(np.float16).view(np.uint16)
    b = (rng.standard_normal(k * n, dtype=np.float32) * s).astype(np.float16).view(np.uint16)
    r = rng.standard_normal(m * n, dtype=np.float32).astype(np.float16).view(np.uint16)
    F16 = kc.DTYPE_F16
    plain = run_dt(backend, a, b, m, k, n, F16)
    want = orc.matmul(a, b, m, k, n, F16)
    if (m, k, n) == (5, 64, 20):
        assert np.array_equal(plain, want)
    else:
        assert norm_max_err(f16_to_f32(plain), f16_to_f32(want)) <= 2e-3
    # fused epilogues act on the narrowed product exactly as the unfused pair
    assert np.array_equal(run_dt(backend, a, b, m, k, n, F16, act=kc.FUSED_SILU), orc.unary_lut(kc.LUT_SILU, F16, plain))
    assert np.array_equal(run_dt(backend, a, b, m, k, n, F16, residual=r), orc.binary(0, plain, r, F16))


@pytest.mark.parametrize("m,k,n", [(8, 256, 64), (33, 100, 20), (64, 512, 128)])
def test_f32_matmul_is_the_reference_recurrence(backend, m, k, n):
    # every f32 product runs the per-cell ascending-k fused-multiply-add chain: bit-exact;
    # the fused activation is the scalar function on the f32 product (no table for 32-bit patterns)
    rng = np.random.default_rng(m * n)
    a = rng.standard_normal(m * k, dtype=np.float32)
    b = rng.standard_normal(k * n, dtype=np.float32) * np.float32(1.0 / np.sqrt(k))
    r = rng.standard_normal(m * n, dtype=np.float32)
    F32 = kc.DTYPE_F32
    assert np.array_equal(run_dt(backend, a, b, m, k, n, F32).view(np.uint32), orc.matmul(a, b, m, k, n, F32).view(np.uint32))
    assert np.array_equal(run_dt(backend, a, b, m, k, n, F32, residual=r).view(np.uint32),
                          orc.matmul(a, b, m, k, n, F32, residual=r).view(np.uint32))
    got = run_dt(backend, a, b, m, k, n, F32, act=kc.FUSED_GELU)
    want = orc.matmul(a, b, m, k, n, F32, act=kc.FUSED_GELU)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
