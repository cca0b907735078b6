"""The peer-memory all-reduce protocol for 2, 4 and 8 ranks on ONE GPU: all ranks run as one
cooperative launch of the same device code, every mailbox in local memory. Every rank must hold the
f32 sum in rank order, truncated to bf16 (then + residual, truncated), bit for bit, call after call."""
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
BF = kc.DTYPE_BF16


def expected(parts, residual=None):
    total = np.float32(0.0) + orc.bf16_to_f32(parts[0])
    for p in parts[1:]:
        total = total + orc.bf16_to_f32(p)
    out = (total.view(np.uint32) >> 16).astype(np.uint16)
    return out if residual is None else orc.binary(0, out, residual, BF)


@pytest.mark.parametrize("world,count", [(2, 64 * 4096), (4, 64 * 4096), (8, 64 * 4096), (8, 64), (3, 12 * 100), (8, 512 * 1024)])
def test_emulated_ranks_agree_bitwise(backend, world, count):
    rng = np.random.default_rng(world * 1000 + count)
    ws = hb.DeviceWorkspace(backend, 3 * world)
    for rep in range(3):                     # consecutive epochs reuse the same mailboxes
        parts = [orc.f32_to_bf16_rne(rng.standard_normal(count).astype(np.float32)) for _ in range(world)]
        res = [orc.f32_to_bf16_rne(rng.standard_normal(count).astype(np.float32)) for _ in range(world)]
        for r in range(world):
            ws.put(r, parts[r])
            ws.put(world + r, res[0])        # the residual stream is replicated
            ws.alloc(2 * world + r, count * 2)
        with_res = rep % 2 == 1
        backend.emulate_all_reduce(ws, list(range(world)), list(range(2 * world, 3 * world)), count, BF,
                                   residual_slots=list(range(world, 2 * world)) if with_res else None, repeats=1)
        want = expected(parts, res[0] if with_res else None)
        for r in range(world):
            assert np.array_equal(ws.read(2 * world + r, count * 2, np.uint16), want), (rep, r)
    # in place, several epochs in one call: out aliases partial, so after k calls every rank holds
    # the k-fold reduction of identical inputs
    parts = [orc.f32_to_bf16_rne(rng.standard_normal(count).astype(np.float32)) for _ in range(world)]
    for r in range(world):
        ws.put(r, parts[r])
    backend.emulate_all_reduce(ws, list(range(world)), list(range(world)), count, BF, repeats=2)
    once = expected(parts)
    twice = expected([once] * world)
    for r in range(world):
        assert np.array_equal(ws.read(r, count * 2, np.uint16), twice)
    ws.close()


def test_refusals(backend):
    ws = hb.DeviceWorkspace(backend, 2)
    ws.alloc(0, 1 << 20)
    ws.alloc(1, 1 << 20)
    with pytest.raises(hb.BackendError):     # count not a multiple of 4 x world
        backend.emulate_all_reduce(ws, [0, 1], [0, 1], 1001, BF)
    with pytest.raises(hb.BackendError):     # message over 1 MiB
        backend.emulate_all_reduce(ws, [0, 1], [0, 1], 1 << 20, BF)
