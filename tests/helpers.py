"""Shared test helpers: seeded input synthesis and dispatch shortcuts."""
import numpy as np

import hologram_b200 as hb
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc

BF16_SPECIALS = np.array(
    [0x0000, 0x8000, 0x7F80, 0xFF80, 0x7FC0, 0xFFC0] + list(range(0x0001, 0x0080)) + list(range(0x8001, 0x8080)),
    dtype=np.uint16)


def f32_to_f16_rne(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def synth_bits(n, dtype, sigma, seed, special_frac=0.0, clamp=None):
    """n seeded draws from N(0, sigma^2) rounded to dtype (RNE: inputs are data), with an
    optional fraction replaced by special bit patterns."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n, dtype=np.float32) * np.float32(sigma)).astype(np.float32)
    if clamp is not None:
        x = np.clip(x, clamp[0], clamp[1])
    bits = orc.f32_to_bf16_rne(x) if dtype == kc.DTYPE_BF16 else f32_to_f16_rne(x)
    if special_frac > 0:
        k = int(n * special_frac)
        pos = rng.choice(n, size=k, replace=False)
        bits[pos] = rng.choice(BF16_SPECIALS, size=k)
    return bits


def synth_bf16(shape, sigma, seed):
    n = int(np.prod(shape))
    return synth_bits(n, kc.DTYPE_BF16, sigma, seed)


def norm_max_err(got_f32, want_f32):
    """max|err| / max|want| — the reference conformance metric (tests/conformance.rs:138-144)."""
    got = np.asarray(got_f32, dtype=np.float64)
    want = np.asarray(want_f32, dtype=np.float64)
    denom = max(np.max(np.abs(want)), 1e-30)
    return float(np.max(np.abs(got - want)) / denom)


def unary(act, inp, out, n, dtype):
    return kc.lut_call(act, kc.UnaryCall(kc.rb(inp) if isinstance(inp, int) else inp,
                                         kc.rb(out) if isinstance(out, int) else out, n, 16, dtype))


# the four legacy-Attention cases of the reference's conformance suite (causal, grouped-query, explicit scale):
# (batch, heads, kv_heads, seq, head_dim, causal, score multiplier or None)
ATTENTION_CASES = ((1, 4, 4, 16, 8, True, None), (2, 8, 2, 12, 16, False, None), (1, 6, 3, 24, 16, True, 0.125), (1, 8, 1, 31, 8, True, None))


def attention_f64(q, k, v, b, h, hkv, s, d, causal, mult):
    """Scaled dot-product attention in float64 (grouped-query, optional causal law)."""
    import numpy as np
    q4 = q.astype(np.float64).reshape(b, h, s, d)
    k4 = np.repeat(k.astype(np.float64).reshape(b, hkv, s, d), h // hkv, axis=1)
    v4 = np.repeat(v.astype(np.float64).reshape(b, hkv, s, d), h // hkv, axis=1)
    div = (1.0 / mult) if mult else max(np.sqrt(d), 1.0)
    sc = np.einsum("bhqd,bhkd->bhqk", q4, k4) / div
    if causal:
        sc = np.where(np.triu(np.ones((s, s), dtype=bool), 1), -np.inf, sc)
    e = np.exp(sc - sc.max(axis=-1, keepdims=True))
    return np.einsum("bhqk,bhkd->bhqd", e / e.sum(axis=-1, keepdims=True), v4).reshape(-1)
