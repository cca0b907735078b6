"""LUT activation dispatch on the GPU, bit-exact against the CPU oracle (through the C ABI)."""
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc
from helpers import synth_bits, unary

pytestmark = pytest.mark.gpu
ACTS = [kc.LUT_SIGMOID, kc.LUT_TANH, kc.LUT_GELU, kc.LUT_SILU, kc.LUT_EXP, kc.LUT_ERF]
DTYPES = [kc.DTYPE_F16, kc.DTYPE_BF16]


def run_lut(backend, act, dtype, bits, in_off=0, out_off=0):
    ws = hb.DeviceWorkspace(backend, 2)
    n = bits.size
    ws.alloc(0, in_off + n * 2)
    ws.alloc(1, out_off + n * 2 + 64)
    ws.write(kc.rb(0, in_off), bits)
    backend.dispatch(unary(act, kc.rb(0, in_off), kc.rb(1, out_off), n, dtype), ws)
    out = ws.read(kc.rb(1, out_off), n * 2, np.uint16)
    guard = ws.read(kc.rb(1, out_off + n * 2), 64)
    assert not guard.any(), "kernel wrote past its output range"
    ws.close()
    return out


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("dtype", DTYPES)
def test_device_built_tables_match_the_oracle(backend, act, dtype):
    assert np.array_equal(backend.lut_table(act, dtype), orc.build_table(act, dtype))


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("dtype", DTYPES)
def test_exhaustive_pass_through_the_kernel(backend, act, dtype):
    allbits = np.arange(65536, dtype=np.uint16)
    assert np.array_equal(run_lut(backend, act, dtype, allbits), orc.build_table(act, dtype))


def test_config1_gelu_bf16_16mi_with_specials(backend):
    n = 16_777_216
    bits = synth_bits(n, kc.DTYPE_BF16, 3.0, 0xC1, special_frac=0.01)
    got = run_lut(backend, kc.LUT_GELU, kc.DTYPE_BF16, bits)
    assert np.array_equal(got, orc.unary_lut(kc.LUT_GELU, kc.DTYPE_BF16, bits))


@pytest.mark.parametrize("act,dtype", [(kc.LUT_SILU, kc.DTYPE_F16), (kc.LUT_EXP, kc.DTYPE_F16), (kc.LUT_ERF, kc.DTYPE_BF16),
                                       (kc.LUT_TANH, kc.DTYPE_BF16), (kc.LUT_SIGMOID, kc.DTYPE_F16)])
def test_sweep_cells_reduced_rows(backend, act, dtype):
    # the [8192, 14336] sweep shape with fewer rows; value law N(0, 4^2), Exp/f16 clamped to [-20, 11]
    n = 512 * 14336
    clamp = (-20.0, 11.0) if (act == kc.LUT_EXP and dtype == kc.DTYPE_F16) else None
    bits = synth_bits(n, dtype, 4.0, 0xC2 + act, clamp=clamp)
    assert np.array_equal(run_lut(backend, act, dtype, bits), orc.unary_lut(act, dtype, bits))


@pytest.mark.parametrize("act,dtype", [(kc.LUT_SILU, kc.DTYPE_BF16), (kc.LUT_TANH, kc.DTYPE_F16), (kc.LUT_EXP, kc.DTYPE_F16),
                                       (kc.LUT_ERF, kc.DTYPE_BF16)])
def test_sweep_cells_full_size(backend, act, dtype):
    # whole [8192, 14336] cells (117,440,512 elements, 470 MB of traffic each), one per dtype plus the
    # clamped f16 Exp cell and an Erf cell, bit-exact over every element
    n = 8192 * 14336
    clamp = (-20.0, 11.0) if (act == kc.LUT_EXP and dtype == kc.DTYPE_F16) else None
    bits = synth_bits(n, dtype, 4.0, 0x2C2 + act, clamp=clamp)
    got = run_lut(backend, act, dtype, bits)
    want = orc.unary_lut(act, dtype, bits)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("n", [1, 7, 8, 9, 255, 4099, (1 << 21) + 5, (1 << 22) + 3])
def test_ragged_sizes(backend, n):
    bits = synth_bits(n, kc.DTYPE_BF16, 3.0, n)
    assert np.array_equal(run_lut(backend, kc.LUT_GELU, kc.DTYPE_BF16, bits),
                          orc.unary_lut(kc.LUT_GELU, kc.DTYPE_BF16, bits))


def test_unaligned_offsets(backend):
    n = (1 << 21) + 11
    bits = synth_bits(n, kc.DTYPE_F16, 2.0, 3)
    got = run_lut(backend, kc.LUT_SILU, kc.DTYPE_F16, bits, in_off=2, out_off=6)
    assert np.array_equal(got, orc.unary_lut(kc.LUT_SILU, kc.DTYPE_F16, bits))


def test_empty_call_is_ok(backend):
    ws = hb.DeviceWorkspace(backend, 2)
    ws.alloc(0, 64)
    ws.alloc(1, 64)
    backend.dispatch(unary(kc.LUT_GELU, 0, 1, 0, kc.DTYPE_BF16), ws)
    backend.synchronize()


def test_short_buffers_fail_loud(backend):
    # cpu/lut.rs:84-92: input shorter than n*2 -> SlotOutOfRange(input), output -> SlotOutOfRange(output)
    ws = hb.DeviceWorkspace(backend, 3)
    ws.alloc(0, 64)
    ws.alloc(1, 128)
    with pytest.raises(hb.BackendError) as e:
        backend.dispatch(unary(kc.LUT_GELU, 0, 1, 64, kc.DTYPE_BF16), ws)
    assert e.value.variant == "SlotOutOfRange" and e.value.slot == 0
    with pytest.raises(hb.BackendError) as e:
        backend.dispatch(unary(kc.LUT_GELU, 1, 0, 64, kc.DTYPE_BF16), ws)
    assert e.value.variant == "SlotOutOfRange" and e.value.slot == 0
    with pytest.raises(hb.BackendError) as e:   # unbound slot
        backend.dispatch(unary(kc.LUT_GELU, 0, 2, 8, kc.DTYPE_BF16), ws)
    assert e.value.slot == 2
    with pytest.raises(hb.BackendError) as e:   # overlapping in/out ranges (split_borrow -> None)
        backend.dispatch(unary(kc.LUT_GELU, kc.rb(1, 0, 64), kc.rb(1, 32, 64), 32, kc.DTYPE_BF16), ws)
    assert e.value.variant == "SlotOutOfRange" and e.value.slot == 1


def test_f64_and_f32_are_refused(backend):
    ws = hb.DeviceWorkspace(backend, 2)
    ws.alloc(0, 1024)
    ws.alloc(1, 1024)
    for dt in (kc.DTYPE_F64, kc.DTYPE_F32):
        with pytest.raises(hb.BackendError) as e:
            backend.dispatch(unary(kc.LUT_GELU, 0, 1, 16, dt), ws)
        assert e.value.variant == "UnsupportedOp"


def test_unknown_variant_is_refused(backend):
    ws = hb.DeviceWorkspace(backend, 2)
    call = kc.KernelCall()
    call.kind = 48   # Conv2d: outside the accelerated path
    with pytest.raises(hb.BackendError) as e:
        backend.dispatch(call, ws)
    assert e.value.variant == "UnsupportedOp"


def test_host_workspace_form(backend):
    # the reference tests' TestWorkspace shape (tests/lut.rs:13-49): host byte slots
    n = 3_000_001
    bits = synth_bits(n, kc.DTYPE_BF16, 3.0, 9)
    out = np.full(n + 8, 0xABCD, dtype=np.uint16)
    ws = hb.HostWorkspace([bits, out])
    backend.dispatch(unary(kc.LUT_GELU, 0, 1, n, kc.DTYPE_BF16), ws)
    got = ws.slots[1].view(np.uint16)
    assert np.array_equal(got[:n], orc.unary_lut(kc.LUT_GELU, kc.DTYPE_BF16, bits))
    assert (got[n:] == 0xABCD).all()


def test_installed_table_is_used(backend):
    t = backend.lut_table(kc.LUT_ERF, kc.DTYPE_BF16)
    try:
        backend.set_lut_table(kc.LUT_ERF, kc.DTYPE_BF16, np.arange(65536, dtype=np.uint16)[::-1].copy())
        bits = synth_bits(100_000, kc.DTYPE_BF16, 1.0, 4)
        got = run_lut(backend, kc.LUT_ERF, kc.DTYPE_BF16, bits)
        assert np.array_equal(got, (65535 - bits.astype(np.int64)).astype(np.uint16))
    finally:
        backend.set_lut_table(kc.LUT_ERF, kc.DTYPE_BF16, t)
