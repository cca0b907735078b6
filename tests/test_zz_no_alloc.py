"""The allocation-free attention entry point against the regular dispatch path (GPU).

`holo_b200_decode_attention_q8_static` is for callers that may not allocate device memory at
call time (an engine that owns all of HBM through its own arena, or one that cannot afford
the implicit device synchronisation of the CUDA allocator): its split-KV partials live in an
array inside the library. Here it is called twice in a row, with different inputs, through the
C ABI with raw device pointers. Each result is checked against the CPU oracle's composition
(Cast / Dequantize / DecodeAttentionValid / Cast) within the 1e-2 tolerance the attention tests
use, and must also equal what `holo_b200_dispatch` produces for the same call (same kernel, same
split count: bit-identical). The second call also shows that whatever the first one left in the
shared array does not leak into later results. The companion status call must report a clean
run.
"""
import ctypes as C

import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from hologram_b200.backend import lib
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

fn = lib.holo_b200_decode_attention_q8_static
fn.restype = C.c_int32
fn.argtypes = [C.c_void_p] * 12 + [C.c_uint32] * 6 + [C.c_uint8]
status_fn = lib.holo_b200_decode_attention_q8_static_status
status_fn.restype = C.c_int32
status_fn.argtypes = [C.c_void_p]


def make_case(b, h, kv, past, d, seed):
    rng = np.random.default_rng(seed)
    q = orc.f32_to_bf16_rne(rng.standard_normal(b * h * d, dtype=np.float32))
    arrs = [q]
    for rows in (b * kv * past, b * kv * past, b * kv, b * kv):
        src = orc.f32_to_bf16_rne(rng.standard_normal(rows * d, dtype=np.float32))
        codes, scales = orc.quantize_rows_i8(src, kc.DTYPE_BF16, rows, d)
        arrs += [codes, scales]
    return arrs


def test_static_scratch_attention_matches_dispatch_twice():
    be = hb.B200Backend(0)
    try:
        for b, h, kv, past, valid, seed in ((4, 32, 8, 2048, 2048, 1), (3, 8, 2, 1156, 700, 2)):
            d = 128
            arrs = make_case(b, h, kv, past, d, seed)
            ws = hb.DeviceWorkspace(be, 12)
            for i, a in enumerate(arrs):
                ws.put(i, a)
            ws.put(9, np.array([valid], dtype=np.uint32))
            ws.alloc(10, b * h * d * 2)
            ws.alloc(11, b * h * d * 2)
            call = kc.DecodeAttentionValidQ8Call(*[kc.rb(i) for i in range(11)], b, h, kv, 1, past, 1, d, 0, kc.DTYPE_BF16)
            be.dispatch(kc.KernelCall.DecodeAttentionValidQ8(call), ws)
            want = ws.read(10, b * h * d * 2, np.uint16).copy()
            ptrs = [ws.slot(i)[0] for i in range(10)] + [ws.slot(11)[0]]
            rc = fn(be.stream, *ptrs, b, h, kv, past, d, 0, kc.DTYPE_BF16)
            assert rc == 0, lib.holo_b200_last_error()
            got = ws.read(11, b * h * d * 2, np.uint16)
            assert status_fn(be.stream) == 0, lib.holo_b200_last_error()
            # the oracle: the reference composition over the same codes and scales
            rc, ref_bits = orc.decode_attention_valid_q8(arrs[0], kc.DTYPE_BF16, *arrs[1:], valid, b, h, kv, 1, past, 1, d, 0)
            assert rc == 0
            ref = orc.bf16_to_f32(ref_bits)
            err = np.max(np.abs(orc.bf16_to_f32(got) - ref)) / np.max(np.abs(ref))
            print(f"static entry point vs oracle: max|err|/max|ref| = {err:.3e}")
            assert err <= 1e-2
            assert np.array_equal(got, want)      # and bit-identical to the dispatch path
            ws.close()
        # a shape whose partials do not fit the built-in array is refused, loudly, before any launch
        rc = fn(be.stream, *([C.c_void_p(256)] * 11), 4096, 32, 8, 65536, 128, 0, kc.DTYPE_BF16)
        assert rc == kc.ERR_UNSUPPORTED_OP and b"built-in" in lib.holo_b200_last_error()
        rc = fn(be.stream, *([C.c_void_p(256)] * 11), 2, 8, 2, 1024, 64, 0, kc.DTYPE_BF16)
        assert rc == kc.ERR_UNSUPPORTED_OP
    finally:
        be.close()
