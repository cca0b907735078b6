"""An encoder-style block made of the calls beyond the decoder's (LayerNorm, MatMul, causal Attention,
BroadcastBinary bias, Relu, Sub, ReduceMean, Expand, Max, Softmax) as one `.holo` archive through the
session, against the CPU interpreter over the same call list: the session's slot sizing, operand
collection and launch order for these variants."""
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import holo
from hologram_b200 import kernel_call as kc
from oracle import interp
from oracle import oracle as orc
from helpers import norm_max_err, synth_bf16

pytestmark = pytest.mark.gpu
BF = kc.DTYPE_BF16


def f32bits(x):
    return int(np.float32(x).view(np.uint32))


def encoder_block(seq=24, d=128, hd=64):
    """x [seq, d] -> LayerNorm -> q / k / v products [seq, hd] -> causal Attention (one head) -> + bias
    (broadcast over rows) -> Relu -> q - that -> row mean -> Expand -> max with the difference -> Softmax."""
    w = holo.HoloWriter()
    names = ["X", "G", "B", "LN", "WQ", "WK", "WV", "Q", "K", "V", "ATT", "BIAS", "BI", "RL", "SB", "MEAN", "EXP", "OUT"]
    S = {n: i for i, n in enumerate(names)}
    n2 = lambda count: count * 2
    rb = lambda name, count: kc.rb(S[name], 0, n2(count))
    consts = {"G": synth_bf16(d, 1.0, 1), "B": synth_bf16(d, 0.1, 2), "BIAS": synth_bf16(hd, 0.5, 6)}
    for i, name in enumerate(("WQ", "WK", "WV")):
        consts[name] = synth_bf16(d * hd, 0.08, 3 + i)
    for name, arr in consts.items():
        w.add_constant(S[name], BF, arr.tobytes())
    w.inputs = [holo.Port("x", S["X"], seq * d, BF, [seq, d])]
    w.outputs = [holo.Port("out", S["OUT"], seq * hd, BF, [seq, hd])]
    sd, sh = seq * d, seq * hd
    calls = [kc.KernelCall.LayerNorm(kc.NormCall(rb("X", sd), rb("G", d), rb("B", d), kc.NONE, rb("LN", sd), seq, d, 0, 0, f32bits(1e-5), BF))]
    for wn, on in (("WQ", "Q"), ("WK", "K"), ("WV", "V")):
        calls.append(kc.KernelCall.MatMul(kc.MatMulCall(rb("LN", sd), rb(wn, d * hd), rb(on, sh), seq, d, hd, BF, 0)))
    calls += [
        # one head of width hd over the whole sequence, causal
        kc.KernelCall.Attention(kc.AttentionCall(rb("Q", sh), rb("K", sh), rb("V", sh), rb("ATT", sh), 1, 1, seq, hd, 0, 1, 0, BF)),
        kc.KernelCall.BroadcastBinary(kc.BroadcastBinaryCall.make(rb("BIAS", hd), rb("ATT", sh), rb("BI", sh), (1, hd), (seq, hd),
                                                                 kc.BROADCAST_ADD, True, BF)),
        kc.KernelCall.Elementwise(kc.K_RELU, kc.UnaryCall(rb("BI", sh), rb("RL", sh), sh, 16, BF)),
        kc.KernelCall.Elementwise(kc.K_SUB, kc.BinaryCall(rb("Q", sh), rb("RL", sh), rb("SB", sh), sh, 16, BF)),
        kc.KernelCall.ReduceMean(kc.ReduceCall.make(rb("SB", sh), rb("MEAN", seq), (seq, hd), 0b10, BF)),
        kc.KernelCall.Expand(kc.ExpandCall.make(rb("MEAN", seq), rb("EXP", sh), (seq, 1), (seq, hd), BF)),
        kc.KernelCall.Elementwise(kc.K_MAX, kc.BinaryCall(rb("EXP", sh), rb("SB", sh), rb("BI", sh), sh, 16, BF)),
        kc.KernelCall.Softmax(kc.SoftmaxCall(rb("BI", sh), rb("OUT", sh), seq, hd, BF)),
    ]
    w.calls = calls
    return w.finish(), S, consts, calls, (seq, d, hd)


def test_encoder_block_session_equals_the_cpu_interpreter(backend):
    img, S, consts, calls, (seq, d, hd) = encoder_block()
    x = synth_bf16(seq * d, 1.0, 42)
    slots = {S[name]: arr.view(np.uint8).reshape(-1).copy() for name, arr in consts.items()}
    slots[S["X"]] = x.view(np.uint8).reshape(-1).copy()
    interp.run(calls, slots)
    want = orc.bf16_to_f32(slots[S["OUT"]][:seq * hd * 2].view(np.uint16))
    for addressed in (False, True):
        sess = hb.InferenceSession(backend, img, addressed=addressed)
        if addressed:
            # inputs reach an addressed walk through the pool, by label; the output is read back by its label
            out_labels, _ = sess.execute_addressed([sess.intern_input(x)])
            got = orc.bf16_to_f32(sess.resolve(out_labels[0], np.uint16))
        else:
            sess.write("x", x)
            sess.execute()
            got = orc.bf16_to_f32(sess.read("out", np.uint16))
        sess.close()
        # tensor-core products and parallel row sums against the CPU's orders: bf16 tolerance
        assert norm_max_err(got, want) <= 2e-2, (addressed, norm_max_err(got, want))
        assert np.allclose(got.reshape(seq, hd).sum(axis=1), 1.0, atol=2e-2)
