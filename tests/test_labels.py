"""Content labels and operation signatures (host only, no GPU): the identity machinery of the
reference's content-addressed executor, restated behind the C ABI.

Pins: the frozen op-signature bytes of `plain_matmul`
(crates/hologram-archive/tests/wire_stability.rs:103-108, 116-125); label shape and sensitivity as
in crates/hologram-archive/src/address.rs:293-330; the digest itself against the independent
Python `blake3` package."""
import json
import os
import struct

import blake3
import numpy as np
import pytest

from hologram_b200 import kernel_call as kc
from hologram_b200 import session as hs


def test_label_of_bytes_is_blake3_hex():
    for data in (b"", b"abc", bytes(range(256)) * 5000):
        lab = hs.label_bytes(np.frombuffer(data, dtype=np.uint8))
        assert len(lab) == 71 and lab == b"blake3:" + blake3.blake3(data).hexdigest().encode()
    assert hs.label_bytes(np.frombuffer(b"abc", np.uint8)) != hs.label_bytes(np.frombuffer(b"abd", np.uint8))


def test_derive_label_folds_opcode_params_and_ordered_operands():
    a = hs.label_bytes(np.arange(10, dtype=np.uint8))
    b = hs.label_bytes(np.arange(11, dtype=np.uint8))
    params = bytes([1, 2, 3])
    got = hs.label_derive(45, params, [a, b])
    assert got == b"blake3:" + blake3.blake3(struct.pack("<H", 45) + params + a + b).hexdigest().encode()
    # order-, opcode- and parameter-sensitive (address.rs:321-330)
    assert hs.label_derive(45, params, [b, a]) != got
    assert hs.label_derive(46, params, [a, b]) != got
    assert hs.label_derive(45, bytes([1, 2, 4]), [a, b]) != got
    assert hs.label_derive(45, params, [a, b]) == got


def test_op_signature_frozen_bytes():
    rb = kc.rb
    mm = kc.MatMulCall(rb(0, 0, 64), rb(1, 0, 64), rb(2, 0, 64), 2, 8, 4, 8, 0)
    assert hs.op_signature(kc.KernelCall.MatMul(mm)) == (45, bytes.fromhex("02000000080000000400000008"))
    # the other variants follow kernel_call.rs:996-1142 / 1321-1516 field for field
    assert hs.op_signature(kc.KernelCall.MatMulActivation(kc.MatMulActivationCall(mm, kc.FUSED_SILU))) == (
        105, bytes.fromhex("02000000080000000400000008") + bytes([kc.FUSED_SILU]))
    assert hs.op_signature(kc.KernelCall.MatMulAdd(kc.MatMulAddCall(mm, rb(3))))[0] == 106
    un = kc.UnaryCall(rb(0), rb(1), 1000, 16, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.Gelu(un)) == (13, struct.pack("<QHB", 1000, 16, kc.DTYPE_BF16))
    assert hs.op_signature(kc.KernelCall.Silu(un))[0] == 14 and hs.op_signature(kc.KernelCall.Erf(un))[0] == 31
    bi = kc.BinaryCall(rb(0), rb(1), rb(2), 77, 16, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.Add(bi)) == (4, struct.pack("<QHB", 77, 16, kc.DTYPE_BF16))
    assert hs.op_signature(kc.KernelCall.Mul(bi))[0] == 6 and hs.op_signature(kc.KernelCall.Concat(bi))[0] == 61
    nc = kc.NormCall(rb(0), rb(1), kc.NONE, kc.NONE, rb(2), 64, 4096, 0, 0, 0x3727C5AC, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.RmsNorm(nc)) == (50, struct.pack("<IIIIQBB", 64, 4096, 0, 0, 0x3727C5AC, kc.DTYPE_BF16, 0))
    nr = kc.NormCall(rb(0), rb(1), kc.NONE, rb(3), rb(2), 64, 4096, 0, 0, 0x3727C5AC, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.AddRmsNorm(nr)) == (53, struct.pack("<IIIIQBB", 64, 4096, 0, 0, 0x3727C5AC, kc.DTYPE_BF16, 1))
    ro = kc.RoPECall(rb(0), rb(1), rb(2), rb(3), 128, 8192, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.RotaryEmbedding(ro)) == (74, struct.pack("<QIB", 8192, 128, kc.DTYPE_BF16))
    tr = kc.TransposeCall.make(rb(0), rb(1), (2, 3, 4), (2, 0, 1), kc.DTYPE_F32)
    assert hs.op_signature(kc.KernelCall.Transpose(tr)) == (60, struct.pack("<BBIBIBIB", 3, kc.DTYPE_F32, 2, 2, 3, 0, 4, 1))
    kv = kc.KvCacheWriteCall(rb(0), rb(1), rb(2), rb(3), 16, 4096, 1, 128)
    assert hs.op_signature(kc.KernelCall.KvCacheWrite(kv)) == (120, struct.pack("<IIII", 16, 4096, 1, 128))
    da = kc.DecodeAttentionValidCall(rb(0), rb(1), rb(2), rb(3), rb(4), rb(5), rb(6), 2, 8, 2, 1, 64, 1, 128, 0, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.DecodeAttentionValid(da)) == (121, struct.pack("<IIIIIIIIB", 2, 8, 2, 1, 64, 1, 128, 0, kc.DTYPE_BF16))
    dm = kc.DecodeAttentionCall(rb(0), rb(1), rb(2), rb(3), rb(4), rb(5), rb(6), 2, 8, 2, 1, 64, 1, 128, 0, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.DecodeAttention(dm))[0] == 119
    ly = kc.LayoutCall(rb(0), rb(1), 99, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.Reshape(ly)) == (59, struct.pack("<QB", 99, kc.DTYPE_BF16))
    assert hs.op_signature(kc.KernelCall.Slice(ly))[0] == 62
    ga = kc.GatherCall(rb(0), rb(1), rb(2), 1, 32000, 4096, 64, kc.DTYPE_I32, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.Gather(ga)) == (114, struct.pack("<QQQQBB", 1, 32000, 4096, 64, kc.DTYPE_I32, kc.DTYPE_BF16))
    ca = kc.CastCall(rb(0), rb(1), 50, kc.DTYPE_BF16, kc.DTYPE_F32)
    assert hs.op_signature(kc.KernelCall.Cast(ca)) == (115, struct.pack("<QBB", 50, kc.DTYPE_BF16, kc.DTYPE_F32))
    ln = kc.NormCall(rb(0), rb(1), rb(2), kc.NONE, rb(3), 4, 64, 0, 0, 0, kc.DTYPE_F32)
    assert hs.op_signature(kc.KernelCall.LayerNorm(ln)) == (49, struct.pack("<IIIIQBB", 4, 64, 0, 0, 0, kc.DTYPE_F32, 0))
    for kind in kc.EXACT_UNARY:
        assert hs.op_signature(kc.KernelCall.Elementwise(kind, kc.UnaryCall(rb(0), rb(1), 9, 0, kc.DTYPE_BF16))) == (kind - 1, struct.pack("<QHB", 9, 0, kc.DTYPE_BF16))
    for kind in kc.EXACT_BINARY:
        assert hs.op_signature(kc.KernelCall.Elementwise(kind, kc.BinaryCall(rb(0), rb(1), rb(2), 9, 0, kc.DTYPE_F32))) == (kind - 1, struct.pack("<QHB", 9, 0, kc.DTYPE_F32))
    dq = kc.DequantActivationCall(rb(0), rb(1), 256, kc.DTYPE_I8, kc.LUT_GELU, kc.DTYPE_F32, 0x3D4CCCCD, -7)
    assert hs.op_signature(kc.KernelCall.DequantActivation(dq)) == (113, struct.pack("<QBBBIi", 256, kc.DTYPE_I8, kc.LUT_GELU, kc.DTYPE_F32, 0x3D4CCCCD, -7))
    wh = kc.WhereCall(rb(0), rb(1), rb(2), rb(3), 77, kc.DTYPE_BF16)
    assert hs.op_signature(kc.KernelCall.Where(wh)) == (77, struct.pack("<QB", 77, kc.DTYPE_BF16))
    at = kc.AttentionCall(rb(0), rb(1), rb(2), rb(3), 1, 8, 31, 8, 1, 1, 0, kc.DTYPE_F32)
    assert hs.op_signature(kc.KernelCall.Attention(at)) == (68, struct.pack("<IIIIIBIB", 1, 8, 31, 8, 1, 1, 0, kc.DTYPE_F32))
    rd = kc.ReduceCall.make(rb(0), rb(1), (3, 4), 0b10, kc.DTYPE_F32)
    assert hs.op_signature(kc.KernelCall.ReduceMax(rd)) == (58, struct.pack("<QBIBBII", 12, 2, 2, 1, kc.DTYPE_F32, 3, 4))
    ex = kc.ExpandCall.make(rb(0), rb(1), (1, 4), (3, 4), kc.DTYPE_F32)
    assert hs.op_signature(kc.KernelCall.Expand(ex)) == (71, struct.pack("<BBIIII", 2, kc.DTYPE_F32, 1, 3, 4, 4))
    bb = kc.BroadcastBinaryCall.make(rb(0), rb(1), rb(2), (1, 4), (3, 4), kc.BROADCAST_SUB, False, kc.DTYPE_F32)
    assert hs.op_signature(kc.KernelCall.BroadcastBinary(bb)) == (112, struct.pack("<BBBBIIII", 2, 1, 0, kc.DTYPE_F32, 1, 3, 4, 4))
    sm = kc.SoftmaxCall(rb(0), rb(1), 64, 4096, kc.DTYPE_F32)
    assert hs.op_signature(kc.KernelCall.Softmax(sm)) == (63, struct.pack("<IIB", 64, 4096, kc.DTYPE_F32))
    # an all-reduce is not a function of local labels: no signature
    import hologram_b200 as hb
    with pytest.raises(hb.BackendError):
        hs.op_signature(kc.KernelCall.AllReduce(kc.AllReduceCall(rb(0), 8, kc.DTYPE_BF16)))


def test_matmul_dequant_signature_and_wire_are_the_frozen_bytes():
    # crates/hologram-archive/tests/wire_stability.rs:57-68, 95-101: output-major W8A8 i8, tag / wire 116
    from hologram_b200 import holo
    buf = lambda i: kc.rb(i, 0, 64)
    c = kc.MatMulDequantCall(buf(0), buf(1), buf(2), buf(3), buf(4), 1, 8, 4, 4, 1, 2, 8, 0, 0, 1, 1, 0, kc.NONE)
    call = kc.KernelCall.MatMulDequant(c)
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.json")))["wire_bytes"]["matmul_dequant_w8a8_omajor"]
    assert hs.op_signature(call) == (golden["signature_opcode"], bytes.fromhex(golden["signature_params_hex"]))
    want = golden["hex"]
    assert holo.encode_calls([call]).hex() == want


def test_matmul_dequant_with_a_codebook_takes_tag_117_and_one_more_byte():
    # kernel_call.rs:1486-1494 (signature), :1589-1598 (codebook operand after the quant operands, before the residual),
    # kernel_codec.rs:525-533 (wire form D_MMDQ3 = the 116 body followed by the codebook reference)
    from hologram_b200 import holo
    buf = lambda i: kc.rb(i, 0, 64)
    c = kc.MatMulDequantCall(buf(0), buf(1), buf(2), buf(3), buf(4), 1, 8, 4, 4, 1, kc.DTYPE_E8CB, 8, 0, 0, 1, 1, 0, kc.NONE)
    plain = holo.encode_calls([kc.KernelCall.MatMulDequant(c)])
    c.codebook = buf(5)
    call = kc.KernelCall.MatMulDequant(c)
    assert call.kind == 117
    op, params = hs.op_signature(call)
    assert op == 117 and params == struct.pack("<IIIIIBBIiBBBB", 1, 8, 4, 4, 1, kc.DTYPE_E8CB, 8, 0, 0, 1, 0, 0, 1)
    wire = holo.encode_calls([call])
    assert wire[4:6] == struct.pack("<H", 117) and wire[6:-20] == plain[6:] and wire[-20:] == struct.pack("<IQQ", 5, 0, 64)


def _b3(data):
    return blake3.blake3(data).digest()


def test_boundary_label_is_the_ordered_product_of_digests():
    # address.rs:197-221 + compose.rs:154-164, computed by hand with the independent blake3 package:
    # op label = address_bytes(opcode LE16 || params); acc = address_bytes(digest(acc) || digest(operand)) per operand
    a = hs.label_bytes(np.arange(10, dtype=np.uint8))
    b = hs.label_bytes(np.arange(11, dtype=np.uint8))
    da, db = _b3(bytes(range(10))), _b3(bytes(range(11)))
    params = bytes([9, 8, 7])
    op = _b3(struct.pack("<H", 45) + params)
    two = _b3(_b3(op + da) + db)
    assert hs.label_derive_boundary(45, params, [a, b]) == b"blake3:" + two.hex().encode()
    # one operand; and no operand at all: the op label composed with itself
    assert hs.label_derive_boundary(45, params, [a]) == b"blake3:" + _b3(op + da).hex().encode()
    assert hs.label_derive_boundary(45, params, []) == b"blake3:" + _b3(op + op).hex().encode()
    # order-sensitive, and a different function of the same pieces than the interior derivation
    assert hs.label_derive_boundary(45, params, [b, a]) != hs.label_derive_boundary(45, params, [a, b])
    assert hs.label_derive_boundary(45, params, [a, b]) != hs.label_derive(45, params, [a, b])
    # a malformed operand label is refused (decode_blake3)
    import hologram_b200 as hb
    with pytest.raises(hb.BackendError):
        hs.label_derive_boundary(45, params, [b"sha256:" + b"0" * 64])
    with pytest.raises(hb.BackendError):
        hs.label_derive_boundary(45, params, [b"blake3:" + b"G" * 64])


def test_matmul_dequant_plain_form_keeps_tag_108_and_wire_111():
    # kernel_call.rs:1475-1500: the all-default form (the [k,n] weight with f32 activations) keeps the base bytes under
    # tag 108; the layout-only bq_omajor does not change the signature; an epilogue or W8A8 takes tag 116
    from hologram_b200 import holo
    buf = lambda i: kc.rb(i, 0, 64)
    c = kc.MatMulDequantCall(buf(0), buf(1), buf(2), buf(3), buf(4), 2, 8, 4, 4, 1, kc.DTYPE_I8, 8, 0x3C000000, -3, 0, 0, 0, kc.NONE)
    call = kc.KernelCall.MatMulDequant(c)
    base = struct.pack("<IIIIIBBIi", 2, 8, 4, 4, 1, kc.DTYPE_I8, 8, 0x3C000000, -3)
    assert call.kind == kc.K_MATMUL_DEQUANT_PLAIN and hs.op_signature(call) == (108, base)
    wire = holo.encode_calls([call])
    assert wire[4:6] == struct.pack("<H", 111) and len(wire) == 4 + 2 + 5 * 20 + len(base)
    c.act = kc.FUSED_SILU
    ext = kc.KernelCall.MatMulDequant(c)
    assert ext.kind == kc.K_MATMUL_DEQUANT and hs.op_signature(ext) == (116, base + bytes([0, kc.FUSED_SILU, 0]))
    c.act, c.residual = 0, buf(5)
    assert hs.op_signature(kc.KernelCall.MatMulDequant(c)) == (116, base + bytes([0, 0, 1]))


def test_matmul_add_activation_signature_and_wire():
    # kernel_call.rs:1469 (opcode 107: matmul parameters then the activation), kernel_codec.rs:519-524 (wire 108)
    from hologram_b200 import holo
    mm = kc.MatMulCall(kc.rb(0, 0, 64), kc.rb(1, 0, 64), kc.rb(2, 0, 64), 2, 8, 4, 8, 0)
    call = kc.KernelCall.MatMulAddActivation(kc.MatMulAddActivationCall(mm, kc.rb(3, 0, 32), kc.FUSED_GELU))
    assert hs.op_signature(call) == (107, bytes.fromhex("02000000080000000400000008") + bytes([kc.FUSED_GELU]))
    wire = holo.encode_calls([call])
    plain = holo.encode_calls([kc.KernelCall.MatMul(mm)])
    assert wire[4:6] == struct.pack("<H", 108) and wire[6:6 + len(plain) - 6] == plain[6:]
    assert wire[-21:] == struct.pack("<IQQB", 3, 0, 32, kc.FUSED_GELU)
