"""Content-addressed execution on the device: resident values are bound by pointer instead of
recomputed, whole-graph repeats are answered from the memo, pool bytes stay bounded
(crates/hologram-exec/src/session.rs:942-984, 1052-1289; crates/hologram-exec/tests/confinement.rs)."""
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import decoder_holo as dh
from hologram_b200 import holo
from hologram_b200 import kernel_call as kc
from hologram_b200 import session as hs
from oracle import oracle as orc
from decoder_common import step_inputs, small_cfg
from helpers import norm_max_err, synth_bf16

pytestmark = pytest.mark.gpu
BF = kc.DTYPE_BF16


def two_branch_archive(m=32, k=256, n=512):
    """out = silu(x @ W1) + z @ W2 with inputs x and z."""
    w = holo.HoloWriter()
    rb = lambda s, nb: kc.rb(s, 0, nb)
    X, Z, W1, W2, Y1, A1, Y2, OUT = range(8)
    w1, w2 = synth_bf16(k * n, 0.05, 1), synth_bf16(k * n, 0.05, 2)
    w.add_constant(W1, BF, w1.tobytes())
    w.add_constant(W2, BF, w2.tobytes())
    w.inputs = [holo.Port("x", X, m * k, BF, [m, k]), holo.Port("z", Z, m * k, BF, [m, k])]
    w.outputs = [holo.Port("out", OUT, m * n, BF, [m, n])]
    w.calls = [
        kc.KernelCall.MatMul(kc.MatMulCall(rb(X, m * k * 2), rb(W1, k * n * 2), rb(Y1, m * n * 2), m, k, n, BF, 0)),
        kc.KernelCall.Silu(kc.UnaryCall(rb(Y1, m * n * 2), rb(A1, m * n * 2), m * n, 16, BF)),
        kc.KernelCall.MatMul(kc.MatMulCall(rb(Z, m * k * 2), rb(W2, k * n * 2), rb(Y2, m * n * 2), m, k, n, BF, 0)),
        kc.KernelCall.Add(kc.BinaryCall(rb(A1, m * n * 2), rb(Y2, m * n * 2), rb(OUT, m * n * 2), m * n, 16, BF)),
    ]
    return w.finish(), (m, k, n, w1, w2)


def expect(x, z, m, k, n, w1, w2):
    a1 = orc.matmul(x, w1, m, k, n, BF, act=kc.FUSED_SILU)
    return orc.binary(0, a1, orc.matmul(z, w2, m, k, n, BF), BF)


def test_subgraph_reuse_memo_and_bounded_pool(backend):
    img, (m, k, n, w1, w2) = two_branch_archive()
    sess = hb.InferenceSession(backend, img, addressed=True)
    x, z1, z2 = (synth_bf16(m * k, 1.0, s) for s in (10, 11, 12))

    def run(x, z):
        sess.write("x", x)
        sess.write("z", z)
        labels, st = sess.execute_addressed([hs.label_bytes(x), hs.label_bytes(z)])
        return labels, st, sess.read("out", np.uint16).copy()

    l1, s1, o1 = run(x, z1)
    # load-time fusion leaves two calls: MatMulActivation(x, W1) and MatMulAdd(z, W2, + that)
    assert sess.n_calls == 2 and (s1.dispatched, s1.skipped, s1.memo_hit) == (2, 0, 0)
    close = lambda got, want: norm_max_err(orc.bf16_to_f32(got), orc.bf16_to_f32(want)) <= 1e-2   # tensor-core sum order
    assert close(o1, expect(x, z1, m, k, n, w1, w2))
    # same inputs: the memo answers, nothing is launched, the output is the resident buffer
    before = backend.launch_count
    l1b, s1b, o1b = run(x, z1)
    assert s1b.memo_hit == 1 and s1b.dispatched == 0 and backend.launch_count == before
    assert l1b == l1 and np.array_equal(o1b, o1)
    # only z changes: the x branch is resident and is bound, not recomputed
    l2, s2, o2 = run(x, z2)
    assert (s2.dispatched, s2.skipped, s2.memo_hit) == (1, 1, 0)
    assert l2 != l1 and close(o2, expect(x, z2, m, k, n, w1, w2)) and not np.array_equal(o2, o1)
    # the labels are the derivation of the fused call list
    lx, lz = hs.label_bytes(x), hs.label_bytes(z2)
    lw1, lw2 = hs.label_bytes(w1), hs.label_bytes(w2)
    op, pr = hs.op_signature(sess.call(0))
    a1 = hs.label_derive(op, pr, [lx, lw1])
    op, pr = hs.op_signature(sess.call(1))
    assert l2[0] == hs.label_derive(op, pr, [lz, lw2, a1])              # operands in kernel order: a, b, residual
    # confinement: alternating inputs for many steps does not grow the pool
    sizes = []
    for step in range(12):
        _, st, _ = run(x, synth_bf16(m * k, 1.0, 100 + step))
        sizes.append(st.pool_bytes)
    assert len(set(sizes[3:])) == 1
    sess.close()


def test_decoder_step_addressed_equals_plain(backend):
    cfg = small_cfg(layers=1, batch=2, bucket=128)
    img, info = dh.build_decoder_step(cfg)
    plain = hb.InferenceSession(backend, img)
    addr = hb.InferenceSession(backend, img, addressed=True)
    vals = step_inputs(cfg, info, 100, 100, seed=5)
    for name, arr in vals.items():
        plain.write(name, arr)
        addr.write(name, arr)
    plain.execute()
    labels, st = addr.execute_addressed([hs.label_bytes(vals[p.name]) for p in addr.inputs])
    assert st.memo_hit == 0 and st.dispatched == addr.n_calls
    assert np.array_equal(addr.read("logits", np.uint16), plain.read("logits", np.uint16))
    for name in ("l0.k_codes_next", "l0.v_scales_next"):
        assert np.array_equal(addr.read(name), plain.read(name))
    assert all(len(l) == 71 and l.startswith(b"blake3:") for l in labels)
    # the same step again is a memo hit with the same labels and the same logits
    labels2, st2 = addr.execute_addressed([hs.label_bytes(vals[p.name]) for p in addr.inputs])
    assert st2.memo_hit == 1 and labels2 == labels
    assert np.array_equal(addr.read("logits", np.uint16), plain.read("logits", np.uint16))
    # a new position only: the embedding / norm / projections of the same tokens are reused
    vals2 = dict(vals)
    vals2["pos"] = np.array([101], dtype=np.int32)
    for name, arr in vals2.items():
        addr.write(name, arr)
    _, st3 = addr.execute_addressed([hs.label_bytes(vals2[p.name]) for p in addr.inputs])
    assert st3.memo_hit == 0 and st3.skipped > 0 and st3.dispatched < addr.n_calls
    plain.close()
    addr.close()
