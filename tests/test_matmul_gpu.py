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


@pytest.mark.parametrize("dtype,m,k,n,act", [(kc.DTYPE_F32, 5, 64, 24, kc.FUSED_GELU), (kc.DTYPE_F32, 3, 33, 17, kc.FUSED_SILU),
                                             (BF, 4, 128, 40, kc.FUSED_TANH), (kc.DTYPE_F16, 6, 72, 16, kc.FUSED_SIGMOID)])
def test_matmul_add_activation_is_the_three_calls(backend, dtype, m, k, n, act):
    # MatMulAddActivation (cpu/float_kernels.rs:899-938): act(A . B + residual) with nothing narrowed between the add and
    # the activation; served on the exact per-cell kernel, so every bit must match. For f32, where the reference forms
    # the triple at load, it is also bit-identical to MatMul -> Add -> activation run separately.
    rng = np.random.default_rng(m * 100 + n)
    if dtype == kc.DTYPE_F32:
        a = rng.standard_normal(m * k, dtype=np.float32) * np.float32(0.2)
        b = rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.2)
        r = rng.standard_normal(m * n, dtype=np.float32)
        store = np.float32
    else:
        narrow = orc.f32_to_bf16_rne if dtype == BF else (lambda x: np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16))
        a, b = narrow(rng.standard_normal(m * k, dtype=np.float32) * np.float32(0.2)), narrow(rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.2))
        r = narrow(rng.standard_normal(m * n, dtype=np.float32))
        store = np.uint16
    es = np.dtype(store).itemsize
    ws = hb.DeviceWorkspace(backend, 4)
    ws.put(0, a)
    ws.put(1, b)
    ws.put(3, r)
    ws.alloc(2, m * n * es)
    mm = kc.MatMulCall(kc.rb(0), kc.rb(1), kc.rb(2), m, k, n, dtype, 0)
    backend.dispatch(kc.KernelCall.MatMulAddActivation(kc.MatMulAddActivationCall(mm, kc.rb(3), act)), ws)
    got = ws.read(2, m * n * es, store)
    want = orc.matmul_add_activation(a, b, r, m, k, n, dtype, act)
    assert np.array_equal(got.view(np.uint32 if es == 4 else np.uint16), want.view(np.uint32 if es == 4 else np.uint16))
    with pytest.raises(hb.BackendError) as e:       # an activation with no table-backed scalar form is refused, loudly
        backend.dispatch(kc.KernelCall.MatMulAddActivation(kc.MatMulAddActivationCall(mm, kc.rb(3), kc.FUSED_RELU)), ws)
    assert e.value.variant == "UnsupportedOp"
    ws.close()


def test_session_forms_the_f32_triple_at_load(backend):
    # fuse_matmul_epilogue (session.rs:2220-2226, 2279-2318): matmul -> add -> activation collapses to one call for f32
    # only; for bf16 the Add is absorbed (MatMulAdd) and the activation stays a call of its own
    from hologram_b200 import holo
    m, k, n = 4, 32, 16
    rng = np.random.default_rng(3)
    outs = {}
    for dtype, store in ((kc.DTYPE_F32, np.float32), (BF, np.uint16)):
        es = np.dtype(store).itemsize
        w = holo.HoloWriter()
        if dtype == BF:
            wt, bias = orc.f32_to_bf16_rne(rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.2)), orc.f32_to_bf16_rne(rng.standard_normal(m * n, dtype=np.float32))
            x = orc.f32_to_bf16_rne(rng.standard_normal(m * k, dtype=np.float32))
        else:
            wt, bias = rng.standard_normal(k * n, dtype=np.float32) * np.float32(0.2), rng.standard_normal(m * n, dtype=np.float32)
            x = rng.standard_normal(m * k, dtype=np.float32)
        w.add_constant(1, dtype, wt.tobytes(), by_reference=False)
        w.add_constant(2, dtype, bias.tobytes(), by_reference=False)
        w.inputs = [holo.Port("x", 0, m * k, dtype, [m, k])]
        w.outputs = [holo.Port("y", 5, m * n, dtype, [m, n])]
        rb = lambda s, cnt: kc.rb(s, 0, cnt * es)
        w.calls = [kc.KernelCall.MatMul(kc.MatMulCall(rb(0, m * k), rb(1, k * n), rb(3, m * n), m, k, n, dtype, 0)),
                   kc.KernelCall.Add(kc.BinaryCall(rb(3, m * n), rb(2, m * n), rb(4, m * n), m * n, 16 if es == 2 else 32, dtype)),
                   kc.KernelCall.Gelu(kc.UnaryCall(rb(4, m * n), rb(5, m * n), m * n, 16 if es == 2 else 32, dtype))]
        w.exec_plan = [[0], [1], [2]]
        if dtype == kc.DTYPE_F32:
            sess = hb.InferenceSession(backend, w.finish())
            assert sess.n_calls == 1 and sess.call(0).kind == kc.K_MATMUL_ADD_ACTIVATION and sess.fused_count == 2
            sess.write("x", x)
            sess.execute()
            got = sess.read("y", np.float32)
            assert np.array_equal(got.view(np.uint32), orc.matmul_add_activation(x, wt, bias, m, k, n, dtype, kc.FUSED_GELU).view(np.uint32))
            sess.close()
        else:
            # a 16-bit Gelu over an Add is a LUT call the session keeps; only the Add is absorbed
            sess = hb.InferenceSession(backend, w.finish())
            assert [sess.call(i).kind for i in range(sess.n_calls)] == [kc.K_MATMUL_ADD, kc.K_GELU]
            sess.close()


@pytest.mark.parametrize("m,k,n,act,res", [(4096, 256, 2560, 0, False), (2500, 320, 2320, kc.FUSED_SILU, False), (2304, 192, 2304, 0, True),
                                           (1333, 128, 8200, 0, False)])
def test_persistent_tile_kernels_within_tolerance(backend, monkeypatch, m, k, n, act, res):
    # shapes with at least one 256 x 256 tile per SM pair take the CTA-pair kernel (tcgen05 cta_group::2), shapes with at
    # least one 128 x 256 tile per SM the one-CTA persistent kernel; ragged edges in both directions, fused epilogues.
    # Both must agree with the CPU chain within the tensor-core tolerance, and with each other and with the
    # one-tile-per-CTA kernel bit for bit (same k order per cell: the accumulation order inside one MMA chain is fixed).
    a, b = synth(m, k, n, m + n)
    r = orc.f32_to_bf16_rne(np.random.default_rng(1).standard_normal(m * n, dtype=np.float32)) if res else None
    want = orc.bf16_to_f32(orc.matmul(a, b, m, k, n, BF, act=act, residual=r))
    outs = {}
    for mode, env in (("pair", {}), ("persistent", {"HOLO_GEMM_PAIR": "0"}), ("classic", {"HOLO_GEMM_PERSISTENT": "0"})):
        for key in ("HOLO_GEMM_PAIR", "HOLO_GEMM_PERSISTENT"):
            monkeypatch.delenv(key, raising=False)
        for key, val in env.items():
            monkeypatch.setenv(key, val)
        outs[mode] = run(backend, a, b, m, k, n, act=act, residual=r)
        err = norm_max_err(orc.bf16_to_f32(outs[mode]), want)
        assert err <= 1e-2, (mode, err)
    backend.synchronize()
    assert np.array_equal(outs["pair"], outs["classic"]) and np.array_equal(outs["persistent"], outs["classic"])
