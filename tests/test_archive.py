"""`.holo` wire format: writer vs the reference's frozen bytes, and the host-only loader checks (no GPU)."""
import json
import os
import struct

import blake3
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import decoder_holo as dh
from hologram_b200 import holo
from hologram_b200 import kernel_call as kc


def test_plain_matmul_wire_bytes_are_the_reference_golden():
    # crates/hologram-archive/tests/wire_stability.rs:103-108
    c = kc.KernelCall.MatMul(kc.MatMulCall(kc.rb(0, 0, 64), kc.rb(1, 0, 64), kc.rb(2, 0, 64), 2, 8, 4, 8, 0))
    want = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))["wire_bytes"]["plain_matmul"]["hex"]
    assert holo.encode_calls([c]).hex() == want


def small_cfg():
    return dh.DecoderConfig(d_model=256, n_heads=2, n_kv_heads=1, head_dim=128, ffn=512, vocab=512, n_layers=1, batch=2, bucket=32)


def test_framing_and_footer():
    img, info = dh.build_decoder_step(small_cfg())
    assert img[:4] == b"HOLO" and struct.unpack("<H", img[4:6])[0] == 3
    assert blake3.blake3(img[:-32]).digest() == img[-32:]        # writer.rs:217-225
    calls, n_in, n_out, n_const = hb.archive_check(img)
    assert calls == info["n_calls"] and n_in == len(info["inputs"]) and n_out == len(info["outputs"])
    assert n_const == len(info["constants"])


def test_corruption_is_refused():
    img, _ = dh.build_decoder_step(small_cfg())
    bad = bytearray(img)
    bad[len(bad) // 2] ^= 1
    with pytest.raises(hb.BackendError) as e:
        hb.archive_check(bytes(bad))
    assert "checksum" in str(e.value) or "fingerprint" in str(e.value)
    with pytest.raises(hb.BackendError):
        hb.archive_check(b"HOLX" + img[4:])
    with pytest.raises(hb.BackendError):
        hb.archive_check(img[:40])
    v9 = bytearray(img)
    v9[4:6] = struct.pack("<H", 9)
    with pytest.raises(hb.BackendError) as e:
        hb.archive_check(bytes(v9), verify=False)
    assert "version" in str(e.value)


def test_unserved_discriminant_is_refused():
    w = holo.HoloWriter()
    body = struct.pack("<IH", 1, 48) + b"\0" * 64          # Conv2d
    img = holo.assemble([(holo.SEC_KERNEL_CALLS, [body]), (holo.SEC_WEIGHTS, [struct.pack("<I", 0)])])
    with pytest.raises(hb.BackendError) as e:
        hb.archive_check(img)
    assert e.value.variant == "UnsupportedOp"


def test_every_served_glue_variant_survives_the_wire():
    # writer (hologram_b200/holo.py) and reader (csrc/archive.cpp) agree on the field order and widths of
    # kernel_codec.rs put_norm / put_softmax / put_reduce / put_expand / put_broadcast_binary / put_transpose
    rb = kc.rb
    calls = [
        kc.KernelCall.LayerNorm(kc.NormCall(rb(0), rb(1), rb(2), kc.NONE, rb(3), 4, 64, 0, 0, 0, kc.DTYPE_F32)),
        kc.KernelCall.Softmax(kc.SoftmaxCall(rb(0), rb(1), 4, 64, kc.DTYPE_F32)),
        kc.KernelCall.ReduceSum(kc.ReduceCall.make(rb(0), rb(1), (4, 8, 2), 0b010, kc.DTYPE_F32)),
        kc.KernelCall.ReduceMax(kc.ReduceCall.make(rb(0), rb(1), (64,), 0, kc.DTYPE_BF16)),
        kc.KernelCall.Expand(kc.ExpandCall.make(rb(0), rb(1), (1, 8), (4, 8), kc.DTYPE_BF16)),
        kc.KernelCall.BroadcastBinary(kc.BroadcastBinaryCall.make(rb(0), rb(1), rb(2), (1, 8), (4, 8), kc.BROADCAST_MUL, True, kc.DTYPE_F32)),
        kc.KernelCall.Transpose(kc.TransposeCall.make(rb(0), rb(1), (2, 3, 4), (2, 0, 1), kc.DTYPE_F32)),
        kc.KernelCall.Attention(kc.AttentionCall(rb(0), rb(1), rb(2), rb(3), 1, 8, 31, 8, 1, 1, 0, kc.DTYPE_F32)),
        kc.KernelCall.DequantActivation(kc.DequantActivationCall(rb(0), rb(1), 256, kc.DTYPE_I8, kc.LUT_GELU, kc.DTYPE_F32, 0x3D4CCCCD, -7)),
        kc.KernelCall.Elementwise(kc.K_DIV, kc.BinaryCall(rb(0), rb(1), rb(2), 9, 0, kc.DTYPE_F32)),
        kc.KernelCall.Elementwise(kc.K_SQRT, kc.UnaryCall(rb(0), rb(1), 9, 0, kc.DTYPE_BF16)),
        kc.KernelCall.Where(kc.WhereCall(rb(0), rb(1), rb(2), rb(3), 9, kc.DTYPE_BF16)),
    ]
    for n in range(1, len(calls) + 1):      # a misread length in call i would derail call i + 1
        img = holo.assemble([(holo.SEC_KERNEL_CALLS, [holo.encode_calls(calls[:n])]), (holo.SEC_WEIGHTS, [struct.pack("<I", 0)])])
        assert hb.archive_check(img)[0] == n


def test_tensor_parallel_shards_partition_the_weights():
    cfg = small_cfg()
    cfg.n_heads, cfg.n_kv_heads = 4, 2
    cfg.d_model = 512
    full = dh.default_weights(cfg)
    _, i0 = dh.build_decoder_step(cfg, 0, 2)
    _, i1 = dh.build_decoder_step(cfg, 1, 2)
    assert i0["heads"] == 2 and i0["kv_heads"] == 1 and i0["ffn"] == cfg.ffn // 2
    # the column shards of wq, concatenated, are the full matrix
    def find(info, nbytes, nth=0):
        hits = [np.frombuffer(bytes(b), dtype=np.uint16) for _, (dt, b) in sorted(info["constants"].items()) if len(b) == nbytes]
        return hits[nth]
    hq = 2 * 128
    a, b = find(i0, 512 * hq * 2).reshape(512, hq), find(i1, 512 * hq * 2).reshape(512, hq)
    assert np.array_equal(np.concatenate([a, b], axis=1), full("l0.wq"))
    # AllReduce precedes each residual add on every rank
    kinds = [c.kind for c in i0["calls"]]
    assert kinds.count(kc.K_ALL_REDUCE) == 2 * cfg.n_layers


def _calls_only(body, extra=()):
    return holo.assemble([(holo.SEC_KERNEL_CALLS, [body]), (holo.SEC_WEIGHTS, [struct.pack("<I", 0)])] + list(extra))


def test_wrapped_weight_length_is_refused():
    # a 64-bit body length near 2^64 must not wrap past the bounds check of the Weights section
    for blen in (0xFFFFFFFFFFFFFFF0, 0xFFFFFFFFFFFFFFFF, 1 << 40):
        weights = struct.pack("<I", 1) + b"\x11" * 32 + struct.pack("<Q", blen) + b"tail"
        img = holo.assemble([(holo.SEC_KERNEL_CALLS, [struct.pack("<I", 0)]), (holo.SEC_WEIGHTS, [weights])])
        with pytest.raises(hb.BackendError) as e:
            hb.archive_check(img, verify=False)
        assert "truncated" in str(e.value)


def test_absurd_slot_numbers_are_refused():
    # slot numbers size the session's tables: one call naming slot 0xFFFFFFFE must not make the loader plan 32 GB
    c = kc.KernelCall.Gelu(kc.UnaryCall(kc.rb(0, 0, 64), kc.rb(0xFFFFFFFE, 0, 64), 32, 16, kc.DTYPE_BF16))
    with pytest.raises(hb.BackendError) as e:
        hb.archive_check(_calls_only(holo.encode_calls([c])), verify=False)
    assert "slot number" in str(e.value)
    ok = kc.KernelCall.Gelu(kc.UnaryCall(kc.rb(0, 0, 64), kc.rb(1, 0, 64), 32, 16, kc.DTYPE_BF16))
    ports = holo.encode_ports([holo.Port("x", 1 << 30, 32, kc.DTYPE_BF16, [32])])
    with pytest.raises(hb.BackendError):
        hb.archive_check(_calls_only(holo.encode_calls([ok]), [(holo.SEC_INPUTS, [ports])]), verify=False)
    assert hb.archive_check(_calls_only(holo.encode_calls([ok])), verify=False)[0] == 1


def test_weightless_archive_needs_a_provider():
    # a constant stored by reference whose body is not in the archive: a plain load must fail loud, never bind
    # the label of empty content (crates/hologram-exec/src/session.rs:669-686)
    w = holo.HoloWriter()
    w.add_constant(0, kc.DTYPE_BF16, bytes(1024), by_reference=True)
    w.calls = [kc.KernelCall.Gelu(kc.UnaryCall(kc.rb(0, 0, 1024), kc.rb(1, 0, 1024), 512, 16, kc.DTYPE_BF16))]
    assert hb.archive_check(w.finish())[3] == 1
    with pytest.raises(hb.BackendError) as e:
        hb.archive_check(w.finish(weightless=True))
    assert "not in the archive" in str(e.value)


def test_new_wire_forms_survive_the_reader():
    rb = kc.rb
    mm = kc.MatMulCall(rb(0, 0, 64), rb(1, 0, 64), rb(2, 0, 64), 2, 8, 4, 8, 0)
    calls = [
        kc.KernelCall.MatMulAddActivation(kc.MatMulAddActivationCall(mm, rb(3, 0, 32), kc.FUSED_GELU)),
        kc.KernelCall.MatMulDequant(kc.MatMulDequantCall(rb(0), rb(1), rb(2), rb(3), rb(4), 2, 8, 4, 4, 1, kc.DTYPE_I8, 8, 0, 0, 0, 0, 0, kc.NONE)),
        kc.KernelCall.MatMulDequant(kc.MatMulDequantCall(rb(0), rb(1), kc.NONE, kc.NONE, rb(4), 2, 8, 4, 0, 1, kc.DTYPE_I4, 8, 0x3C000000, 1, 0, 0, kc.FUSED_TANH, rb(5))),
        kc.KernelCall.Softmax(kc.SoftmaxCall(rb(0), rb(1), 4, 64, kc.DTYPE_F32)),
    ]
    assert [c.kind for c in calls[:3]] == [108, 111, 116]
    for n in range(1, len(calls) + 1):
        assert hb.archive_check(_calls_only(holo.encode_calls(calls[:n])), verify=False)[0] == n
