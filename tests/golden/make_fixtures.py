"""Writes tests/golden/oracle_fixtures.json: BLAKE3 digests of CPU-oracle outputs on small seeded inputs.

Run from the repository root:  python tests/golden/make_fixtures.py
`compute()` is also imported by tests/test_golden.py, which checks that the oracle still produces
exactly these bits."""
import json
import os
import sys

import blake3
import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from hologram_b200 import kernel_call as kc  # noqa: E402
from oracle import oracle as orc  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_fixtures.json")
BF, F16, F32 = kc.DTYPE_BF16, kc.DTYPE_F16, kc.DTYPE_F32


def digest(*arrays):
    h = blake3.blake3()
    for a in arrays:
        h.update(np.ascontiguousarray(a).view(np.uint8).tobytes())
    return h.hexdigest()


def f32bits(x):
    return int(np.float32(x).view(np.uint32))


def compute():
    out = {}
    codes = np.arange(65536, dtype=np.uint16)
    for name, act in (("sigmoid", kc.LUT_SIGMOID), ("tanh", kc.LUT_TANH), ("gelu", kc.LUT_GELU), ("silu", kc.LUT_SILU)):
        for dn, dt in (("f16", F16), ("bf16", BF)):
            out[f"lut_table_{name}_{dn}"] = digest(orc.unary_lut(act, dt, codes))
    rng = np.random.default_rng(2024)
    x = (rng.standard_normal(8 * 160) * 3).astype(np.float32)
    xb = orc.f32_to_bf16_rne(x)
    g = orc.f32_to_bf16_rne(rng.standard_normal(160).astype(np.float32))
    out["quantize_rows_i8_bf16"] = digest(*orc.quantize_rows_i8(xb, BF, 8, 160))
    out["rms_norm_bf16"] = digest(orc.rms_norm(xb, g, 8, 160, f32bits(1e-5), BF))
    out["add_rms_norm_bf16"] = digest(orc.add_rms_norm(xb, xb[::-1].copy(), g, 8, 160, f32bits(1e-5), BF))
    out["layer_norm_f32"] = digest(orc.layer_norm(x, None, None, 8, 160, 0, F32))
    out["softmax_f32"] = digest(orc.softmax(x, 8, 160, F32))
    out["reduce_sum_axis1_bf16"] = digest(orc.reduce(xb, (8, 160), 0b10, 0, False, BF))
    out["elementwise_div_f32"] = digest(orc.elementwise(kc.K_DIV, x, x[::-1].copy(), F32))
    out["elementwise_round_bf16_all_codes"] = digest(orc.elementwise(kc.K_ROUND, codes, None, BF))
    m, k, n = 5, 96, 40
    a = orc.f32_to_bf16_rne(rng.standard_normal(m * k).astype(np.float32))
    b = orc.f32_to_bf16_rne((rng.standard_normal(k * n) * 0.1).astype(np.float32))
    out["matmul_bf16"] = digest(orc.matmul(a, b, m, k, n, BF))
    out["matmul_silu_bf16"] = digest(orc.matmul(a, b, m, k, n, BF, act=kc.FUSED_SILU))
    bsz, h, kv, past, d = 2, 4, 2, 37, 32
    q, kp, vp, kn, vn = (rng.standard_normal(c).astype(np.float32) for c in (bsz * h * d, bsz * kv * past * d, bsz * kv * past * d, bsz * kv * d, bsz * kv * d))
    rc, att = orc.decode_attention_valid(q, kp, vp, kn, vn, 29, bsz, h, kv, 1, past, 1, d, 0, F32)
    assert rc == 0
    out["decode_attention_valid_f32"] = digest(att)
    aq, ak, av = (rng.standard_normal(c).astype(np.float32) for c in (2 * 12 * 16, 12 * 16, 12 * 16))
    out["attention_causal_f32"] = digest(orc.attention(aq, ak, av, 1, 2, 1, 12, 16, True, 0, F32))   # 2 q heads on 1 kv head, seq 12
    m, k, n = 3, 128, 17
    af = rng.standard_normal(m * k).astype(np.float32)
    sc = (rng.random(n).astype(np.float32) + np.float32(0.01)) * np.float32(0.02)
    out["w8a8_i8"] = digest(orc.matmul_w8a8_omajor(af, rng.integers(-127, 128, size=n * k, dtype=np.int8), sc, m, k, n))
    out["w4a8_i4"] = digest(orc.matmul_w8a8_omajor(af, rng.integers(0, 256, size=n * k // 2, dtype=np.uint8), sc, m, k, n, i4=True))
    out["w1a8_e8cb"] = digest(orc.matmul_w8a8_omajor(af, rng.integers(0, 256, size=n * k // 8, dtype=np.uint8), sc, m, k, n,
                                                     codebook=rng.integers(-127, 128, size=2048, dtype=np.int8)))
    out["dequant_activation_i8_gelu"] = digest(orc.dequant_activation(np.arange(256, dtype=np.uint8), 256, kc.DTYPE_I8, kc.LUT_GELU, np.float32(0.05), -7))
    return out


if __name__ == "__main__":
    with open(OUT, "w") as f:
        json.dump(compute(), f, indent=2, sort_keys=True)
    print("wrote", OUT)
