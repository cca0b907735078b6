"""Shared pieces of the decoder tests: deterministic inputs for one decode step."""
import numpy as np

from hologram_b200 import decoder_holo as dh
from hologram_b200 import kernel_call as kc
from oracle import oracle as orc


def small_cfg(layers=2, batch=4, bucket=160):
    return dh.DecoderConfig(d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=1024, n_layers=layers,
                            batch=batch, bucket=bucket)


def step_inputs(cfg, info, position, valid_len, seed=0, tp_rank=0):
    """name -> numpy array for every input port of one rank's archive. The KV cache content is
    the quantizer applied to seeded N(0,1) rows (so codes/scales are a realistic cache)."""
    rng = np.random.default_rng(seed)
    H, KV, hd, B = info["heads"], info["kv_heads"], cfg.head_dim, cfg.batch
    vals = {"token_ids": rng.integers(0, cfg.vocab, size=B).astype(np.int32),
            "pos": np.array([position % (1 << 32)], dtype=np.uint32).view(np.int32),
            "valid_len": np.array([valid_len], dtype=np.uint32).view(np.int32)}
    vals["cos_q"], vals["sin_q"] = dh.rope_tables(cfg, position, H)
    vals["cos_k"], vals["sin_k"] = dh.rope_tables(cfg, position, KV)
    rows = B * KV * cfg.bucket
    for l in range(cfg.n_layers):
        for which in ("k", "v"):
            r2 = np.random.default_rng([seed, l, ord(which), tp_rank])
            src = orc.f32_to_bf16_rne(r2.standard_normal(rows * hd, dtype=np.float32))
            codes, scales = orc.quantize_rows_i8(src, kc.DTYPE_BF16, rows, hd)
            vals[f"l{l}.{which}_codes"], vals[f"l{l}.{which}_scales"] = codes, scales
    return vals


def oracle_step(info, vals, all_reduce=None):
    """Run the unfused call list on the CPU interpreter; returns the slot dict."""
    from oracle import interp
    slots = {s: np.frombuffer(bytes(body), dtype=np.uint8).copy() for s, (dt, body) in info["constants"].items()}
    for p in info["inputs"]:
        slots[p.slot] = np.ascontiguousarray(vals[p.name]).view(np.uint8).reshape(-1).copy()
    interp.run(info["calls"], slots, all_reduce=all_reduce)
    return slots
