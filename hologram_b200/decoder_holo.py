"""Builds the decode-step `.holo` of a Llama-style decoder from KernelCalls.

The reference compiler (crates/hologram-compiler) needs its Rust toolchain, so archives for
this path are written directly in its wire format. The call list is what the compiler's
lowering produces for one decode step after `desugar_composites`
(crates/hologram-graph/src/graph.rs:428-456: FusedSwiGlu -> MatMul, Silu, MatMul, Mul), with
the KV writes deferred to a trailing level (crates/hologram-compiler/src/compiler.rs:180-219),
plus the extension calls of this backend (row quantizer, int8-KV attention, all-reduce).
MatMul -> Silu and MatMul -> Add pairs are emitted unfused; the session fuses them at load.

Tensor parallel: rank r of G holds heads/G query heads, kv_heads/G KV heads and ffn/G FFN
columns; q/k/v/gate/up are column shards, o/down are row shards followed by an AllReduce and
the residual Add; the LM head is a vocabulary-column shard (each rank returns its slice of the
logits, no gather); norms, the embedding and the residual stream are replicated.
"""
import struct

import numpy as np

from . import holo
from . import kernel_call as kc

BF, I8, F32, I32, U32_AS = kc.DTYPE_BF16, kc.DTYPE_I8, kc.DTYPE_F32, kc.DTYPE_I32, kc.DTYPE_I32


class DecoderConfig:
    def __init__(self, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, vocab=32000, n_layers=8,
                 batch=64, bucket=4096, eps=1e-5, rope_theta=10000.0):
        self.d_model, self.n_heads, self.n_kv_heads, self.head_dim = d_model, n_heads, n_kv_heads, head_dim
        self.ffn, self.vocab, self.n_layers, self.batch, self.bucket = ffn, vocab, n_layers, batch, bucket
        self.eps, self.rope_theta = eps, rope_theta


def _f32_bits(x):
    return struct.unpack("<I", struct.pack("<f", x))[0]


def bf16_rne(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def default_weights(cfg, seed=0xC5):
    """name -> bf16 bit array, N(0, 0.02^2) (norm gains are 1 + N(0, 0.02^2)), seeded per tensor."""
    def gen(name, shape, gain=False):
        rng = np.random.default_rng([seed, abs(hash(name)) % (1 << 31)] if False else [seed] + [ord(c) for c in name])
        w = rng.standard_normal(int(np.prod(shape)), dtype=np.float32) * np.float32(0.02)
        if gain:
            w += np.float32(1.0)
        return bf16_rne(w).reshape(shape)
    d, hq, hkv, f = cfg.d_model, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim, cfg.ffn
    def get(name):
        layer_shapes = {"wq": (d, hq), "wk": (d, hkv), "wv": (d, hkv), "wo": (hq, d), "wg": (d, f), "wu": (d, f), "wd": (f, d)}
        base = name.split(".")[-1]
        if base in ("g1", "g2", "gf"):
            return gen(name, (d,), gain=True)
        if base == "embed":
            return gen(name, (cfg.vocab, d))
        if base == "lm_head":
            return gen(name, (d, cfg.vocab))
        return gen(name, layer_shapes[base])
    return get


def rope_tables(cfg, position, heads):
    """cos/sin with x's element layout [batch, heads, 1, head_dim] (rotate-half form,
    float_kernels.rs:3123-3190), every sequence at the same position."""
    half = cfg.head_dim // 2
    inv = cfg.rope_theta ** (-np.arange(half, dtype=np.float64) / half)
    ang = position * inv
    c = np.concatenate([np.cos(ang), np.cos(ang)]).astype(np.float32)
    s = np.concatenate([np.sin(ang), np.sin(ang)]).astype(np.float32)
    tile = lambda v: np.tile(bf16_rne(v), cfg.batch * heads)
    return tile(c), tile(s)


class _Slots:
    def __init__(self):
        self.n = 0
        self.bytes = {}

    def new(self, nbytes):
        s = self.n
        self.n += 1
        self.bytes[s] = nbytes
        return s


def build_decoder_step(cfg, tp_rank=0, tp_world=1, weights=None, seed=0xC5):
    """Returns (archive_bytes, info) for one decode step of rank `tp_rank` of `tp_world`."""
    G = tp_world
    assert cfg.n_heads % G == 0 and cfg.n_kv_heads % G == 0 and cfg.ffn % G == 0 and cfg.vocab % G == 0
    W = weights or default_weights(cfg, seed)
    B, d, hd = cfg.batch, cfg.d_model, cfg.head_dim
    H, KV, F, V = cfg.n_heads // G, cfg.n_kv_heads // G, cfg.ffn // G, cfg.vocab // G
    hq, hkv = H * hd, KV * hd
    w = holo.HoloWriter()
    sl = _Slots()
    calls, trailing = [], []
    rb = lambda s: kc.rb(s, 0, sl.bytes[s])

    def const(arr, dtype):
        a = np.ascontiguousarray(arr)
        s = sl.new(a.nbytes)
        w.add_constant(s, dtype, a.view(np.uint8).reshape(-1).data, by_reference=a.nbytes > 256)
        return s

    def inp(name, nbytes, count, dtype, shape):
        s = sl.new(nbytes)
        w.inputs.append(holo.Port(name, s, count, dtype, shape))
        return s

    col = lambda m, n: np.ascontiguousarray(m[:, tp_rank * n:(tp_rank + 1) * n])
    row = lambda m, n: np.ascontiguousarray(m[tp_rank * n:(tp_rank + 1) * n, :])

    ids = inp("token_ids", B * 4, B, I32, [B])
    pos = inp("pos", 4, 1, I32, [1])
    valid = inp("valid_len", 4, 1, I32, [1])
    cos_q = inp("cos_q", B * hq * 2, B * hq, BF, [B, H, 1, hd])
    sin_q = inp("sin_q", B * hq * 2, B * hq, BF, [B, H, 1, hd])
    cos_k = inp("cos_k", B * hkv * 2, B * hkv, BF, [B, KV, 1, hd])
    sin_k = inp("sin_k", B * hkv * 2, B * hkv, BF, [B, KV, 1, hd])

    def matmul(a, b, m, k, n):
        o = sl.new(m * n * 2)
        calls.append(kc.KernelCall.MatMul(kc.MatMulCall(rb(a), rb(b), rb(o), m, k, n, BF, 0)))
        return o

    def rms(x, g):
        o = sl.new(B * d * 2)
        calls.append(kc.KernelCall.RmsNorm(kc.NormCall(rb(x), rb(g), kc.NONE, kc.NONE, rb(o), B, d, 0, 0, _f32_bits(cfg.eps), BF)))
        return o

    def add(a, b, n):
        o = sl.new(n * 2)
        calls.append(kc.KernelCall.Add(kc.BinaryCall(rb(a), rb(b), rb(o), n, 16, BF)))
        return o

    def reduce_then_add(partial, residual, n):
        if G > 1:
            calls.append(kc.KernelCall.AllReduce(kc.AllReduceCall(rb(partial), n, BF)))
        return add(partial, residual, n)

    x = sl.new(B * d * 2)
    emb = const(W("embed"), BF)
    calls.append(kc.KernelCall.Gather(kc.GatherCall(rb(emb), rb(ids), rb(x), 1, cfg.vocab, d, B, I32, BF)))
    rows_cache = B * KV * cfg.bucket
    for l in range(cfg.n_layers):
        p = f"l{l}."
        h = rms(x, const(W(p + "g1"), BF))
        q = matmul(h, const(col(W(p + "wq"), hq), BF), B, d, hq)
        k = matmul(h, const(col(W(p + "wk"), hkv), BF), B, d, hkv)
        v = matmul(h, const(col(W(p + "wv"), hkv), BF), B, d, hkv)
        qr, kr = sl.new(B * hq * 2), sl.new(B * hkv * 2)
        calls.append(kc.KernelCall.RotaryEmbedding(kc.RoPECall(rb(q), rb(cos_q), rb(sin_q), rb(qr), hd, B * hq, BF)))
        calls.append(kc.KernelCall.RotaryEmbedding(kc.RoPECall(rb(k), rb(cos_k), rb(sin_k), rb(kr), hd, B * hkv, BF)))
        kcod, ksc, vcod, vsc = sl.new(B * hkv), sl.new(B * KV * 4), sl.new(B * hkv), sl.new(B * KV * 4)
        calls.append(kc.KernelCall.QuantizeRowsI8(kc.QuantizeRowsI8Call(rb(kr), rb(kcod), rb(ksc), B * KV, hd, BF)))
        calls.append(kc.KernelCall.QuantizeRowsI8(kc.QuantizeRowsI8Call(rb(v), rb(vcod), rb(vsc), B * KV, hd, BF)))
        cache = {}
        for nm, rbytes, dt in (("k_codes", hd, I8), ("k_scales", 4, F32), ("v_codes", hd, I8), ("v_scales", 4, F32)):
            count = rows_cache * (hd if dt == I8 else 1)
            shape = [B, KV, cfg.bucket, hd] if dt == I8 else [B, KV, cfg.bucket]
            cache[nm] = inp(f"{p}{nm}", rows_cache * rbytes, count, dt, shape)
        att = sl.new(B * hq * 2)
        calls.append(kc.KernelCall.DecodeAttentionValidQ8(kc.DecodeAttentionValidQ8Call(
            rb(qr), rb(cache["k_codes"]), rb(cache["k_scales"]), rb(cache["v_codes"]), rb(cache["v_scales"]),
            rb(kcod), rb(ksc), rb(vcod), rb(vsc), rb(valid), rb(att), B, H, KV, 1, cfg.bucket, 1, hd, 0, BF)))
        o = matmul(att, const(row(W(p + "wo"), hq), BF), B, hq, d)
        x = reduce_then_add(o, x, B * d)
        h2 = rms(x, const(W(p + "g2"), BF))
        gate = matmul(h2, const(col(W(p + "wg"), F), BF), B, d, F)
        act = sl.new(B * F * 2)
        calls.append(kc.KernelCall.Silu(kc.UnaryCall(rb(gate), rb(act), B * F, 16, BF)))
        up = matmul(h2, const(col(W(p + "wu"), F), BF), B, d, F)
        gu = sl.new(B * F * 2)
        calls.append(kc.KernelCall.Mul(kc.BinaryCall(rb(act), rb(up), rb(gu), B * F, 16, BF)))
        dn = matmul(gu, const(row(W(p + "wd"), F), BF), B, F, d)
        x = reduce_then_add(dn, x, B * d)
        # KV appends: deferred to the trailing level, written at the runtime position
        for nm, newslot, rbytes, dt in (("k_codes", kcod, hd, I8), ("k_scales", ksc, 4, F32), ("v_codes", vcod, hd, I8), ("v_scales", vsc, 4, F32)):
            out = sl.new(rows_cache * rbytes)
            count = rows_cache * (hd if dt == I8 else 1)
            shape = [B, KV, cfg.bucket, hd] if dt == I8 else [B, KV, cfg.bucket]
            w.outputs.append(holo.Port(f"{p}{nm}_next", out, count, dt, shape))
            trailing.append(kc.KernelCall.KvCacheWrite(kc.KvCacheWriteCall(rb(cache[nm]), rb(newslot), rb(pos), rb(out), B * KV, cfg.bucket, 1, rbytes)))
    hf = rms(x, const(W("gf"), BF))
    logits = matmul(hf, const(col(W("lm_head"), V), BF), B, d, V)
    w.outputs.insert(0, holo.Port("logits", logits, B * V, BF, [B, V]))
    w.calls = calls + trailing
    w.exec_plan = [[i] for i in range(len(calls))] + [list(range(len(calls), len(calls) + len(trailing)))]
    info = {"n_calls": len(w.calls), "heads": H, "kv_heads": KV, "ffn": F, "vocab": V, "calls": w.calls,
            "inputs": w.inputs, "outputs": w.outputs, "slot_bytes": dict(sl.bytes),
            "constants": {s: (dt, body) for s, dt, body in w.inline_constants + w.weight_constants}}
    return w.finish(), info
