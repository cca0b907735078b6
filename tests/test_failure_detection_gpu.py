"""Failure detection without faulting a GPU: every device-side wait is bounded and reports to the host;
the tensor-parallel group's set-up has a host-side time limit. Nothing here traps, hangs or faults:
the "failure" is a peer that never sends (an emulated rank whose CTAs return at once) and a rank
that never joins (a group of two with only one member present)."""
import time

import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc
from helpers import synth_bits, unary

pytestmark = pytest.mark.gpu
BF = kc.DTYPE_BF16


def test_a_peer_that_never_sends_surfaces_as_dispatch_error_and_the_context_survives():
    be = hb.B200Backend(0)
    try:
        world, count = 4, 16 * 1024
        rng = np.random.default_rng(1)
        ws = hb.DeviceWorkspace(be, 2 * world)
        parts = [orc.f32_to_bf16_rne(rng.standard_normal(count).astype(np.float32)) for _ in range(world)]
        for r in range(world):
            ws.put(r, parts[r])
            ws.alloc(world + r, count * 2)
        t0 = time.time()
        with pytest.raises(hb.BackendError) as e:
            be.emulate_all_reduce(ws, list(range(world)), list(range(world, 2 * world)), count, BF, withheld_rank=2, poll_limit=1 << 12)
        assert e.value.variant == "Dispatch" and "bounded wait" in str(e.value)
        assert time.time() - t0 < 30.0            # the polls ran out; nobody waited for ever
        # the status was consumed by the report: the same call with every rank present now works, bit for bit
        be.emulate_all_reduce(ws, list(range(world)), list(range(world, 2 * world)), count, BF)
        total = np.float32(0.0) + orc.bf16_to_f32(parts[0])
        for p in parts[1:]:
            total = total + orc.bf16_to_f32(p)
        want = (total.view(np.uint32) >> 16).astype(np.uint16)
        for r in range(world):
            assert np.array_equal(ws.read(world + r, count * 2, np.uint16), want)
        # and an unrelated kernel runs
        bits = synth_bits(100_000, BF, 3.0, 2)
        ws2 = hb.DeviceWorkspace(be, 2)
        ws2.put(0, bits)
        ws2.alloc(1, bits.nbytes)
        be.dispatch(unary(kc.LUT_GELU, 0, 1, bits.size, BF), ws2)
        assert np.array_equal(ws2.read(1, bits.nbytes, np.uint16), orc.unary_lut(kc.LUT_GELU, BF, bits))
    finally:
        be.close()


def test_a_rank_that_never_joins_is_a_host_timeout():
    # a tensor-parallel group of two with one member: the non-blocking set-up is polled on the host and aborted
    # after the limit; nothing was enqueued on the GPU, the context keeps working
    be = hb.B200Backend(0)
    try:
        uid = hb.B200Backend.nccl_unique_id()
        t0 = time.time()
        with pytest.raises(hb.BackendError) as e:
            be.init_tp(uid, 0, 2, timeout_ms=3000)
        waited = time.time() - t0
        assert e.value.variant == "Init" and "did not form" in str(e.value)
        assert 2.0 <= waited < 60.0
        assert be.tp_transport == 0
        bits = synth_bits(50_000, BF, 3.0, 3)
        ws = hb.DeviceWorkspace(be, 2)
        ws.put(0, bits)
        ws.alloc(1, bits.nbytes)
        be.dispatch(unary(kc.LUT_SILU, 0, 1, bits.size, BF), ws)
        assert np.array_equal(ws.read(1, bits.nbytes, np.uint16), orc.unary_lut(kc.LUT_SILU, BF, bits))
    finally:
        be.close()
