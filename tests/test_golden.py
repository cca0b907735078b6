"""The committed golden files: the CPU oracle still produces the frozen bits (tests/golden/oracle_fixtures.json,
written by tests/golden/make_fixtures.py), and the reference-held vectors file is well formed."""
import json
import os
import sys

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_oracle_reproduces_the_committed_fixtures():
    sys.path.insert(0, GOLDEN)
    import make_fixtures
    want = json.load(open(os.path.join(GOLDEN, "oracle_fixtures.json")))
    got = make_fixtures.compute()
    assert set(got) == set(want)
    moved = [k for k in want if got[k] != want[k]]
    assert not moved, moved


def test_reference_vectors_file_names_its_sources():
    d = json.load(open(os.path.join(GOLDEN, "reference_vectors.json")))
    assert all(int(d["fnv1a64_of_output_bits"][k], 16) > 0 for k in ("i8_w8a8", "i4_w4a8", "e8cb_w1a8"))
    for entry in d["wire_bytes"].values():
        assert "crates/hologram-archive/tests/wire_stability.rs" in entry["source"] and bytes.fromhex(entry["hex"])


import numpy as np
import pytest


@pytest.mark.gpu
def test_gpu_lut_tables_equal_the_committed_digests(backend):
    # the device path against the committed fixture itself (not only against the live oracle)
    import blake3
    import hologram_b200 as hb
    from hologram_b200 import kernel_call as kc
    want = json.load(open(os.path.join(GOLDEN, "oracle_fixtures.json")))
    codes = np.arange(65536, dtype=np.uint16)
    for name, ctor in (("sigmoid", kc.KernelCall.Sigmoid), ("tanh", kc.KernelCall.Tanh), ("gelu", kc.KernelCall.Gelu), ("silu", kc.KernelCall.Silu)):
        for dn, dt in (("f16", kc.DTYPE_F16), ("bf16", kc.DTYPE_BF16)):
            ws = hb.DeviceWorkspace(backend, 2)
            ws.put(0, codes)
            ws.alloc(1, codes.nbytes)
            backend.dispatch(ctor(kc.UnaryCall(kc.rb(0), kc.rb(1), codes.size, 16, dt)), ws)
            got = np.ascontiguousarray(ws.read(1, codes.nbytes, np.uint16))
            ws.close()
            assert blake3.blake3(got.view(np.uint8).tobytes()).hexdigest() == want[f"lut_table_{name}_{dn}"], (name, dn)
