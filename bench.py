#!/usr/bin/env python
"""Benchmark of the B200 backend hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload lut|lut_sweep|attention|matmul|gemv|w8a8|decoder]
  python bench.py --impl reference ...      # the reference CPU path (oracle restatement) on host cores

One JSON line on stdout (rank 0). Timed with CUDA events on the stream the kernels are
launched on; inputs are larger than L2 or rotated over buffers larger than L2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML read-only queries from a thread
    every few milliseconds (nvidia-smi in a loop, far coarser, only if NVML cannot be loaded)."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index, uuid=None):
        self.index, self.uuid, self.rows, self.proc = index, uuid, [], None
        self.nvml, self.handle, self.thread, self.stop_flag = None, None, None, False
        self.sm, self.mask, self.sm_max = [], 0, None

    def _nvml_open(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = None
            if self.uuid:
                for cand in (self.uuid, "GPU-" + self.uuid):
                    try:
                        h = pynvml.nvmlDeviceGetHandleByUUID(cand.encode() if isinstance(cand, str) else cand)
                        break
                    except Exception:
                        h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self.nvml, self.handle = pynvml, h
            return True
        except Exception:
            self.nvml = None
            return False

    def _poll(self):
        n, h = self.nvml, self.handle
        reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag:
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)))
                self.mask |= int(reasons(h))
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self._nvml_open():
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.thread:
            self.stop_flag = True
            self.thread.join(timeout=1.0)
            reasons = sorted(name for bit, name in self.REASON_BITS.items() if self.mask & bit)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.sm_max,
                    "reasons": reasons, "samples": len(self.sm), "source": "nvml"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "source": "nvidia-smi"}


# ------------------------------------------------------------------------------------------
# Workloads. Each returns a dict: run_device(step), run_host(step) (end-to-end through the
# host-workspace C-ABI call), units per step, algorithmic bytes (or flops) per launch of the
# dominant kernel, and a cpu_baseline callable.
# ------------------------------------------------------------------------------------------

def bf16_rne(x):
    from hologram_b200 import decoder_holo as dh
    return dh.bf16_rne(x)


def synth_c1(n, seed):
    """Config 1 input law: 99% N(0, 3^2) rounded to bf16, 1% special bit patterns."""
    rng = np.random.default_rng(seed)
    bits = bf16_rne((rng.standard_normal(n, dtype=np.float32) * np.float32(3.0)))
    special = np.array([0x0000, 0x8000, 0x7F80, 0xFF80, 0x7FC0, 0xFFC0] + list(range(1, 0x80)) +
                       list(range(0x8001, 0x8080)), dtype=np.uint16)
    k = n // 100
    bits[rng.choice(n, size=k, replace=False)] = rng.choice(special, size=k)
    return bits


def workload_lut(be, torch, rank, args):
    import hologram_b200 as hb
    from hologram_b200 import kernel_call as kc
    n = 16_777_216
    pairs = 8  # 8 x (32 MiB in + 32 MiB out) = 512 MiB rotated: every step misses the 126 MB L2
    host_in = torch.from_numpy(synth_c1(n, 0xC1 + rank).view(np.int16)).pin_memory()
    host_out = torch.empty(n, dtype=torch.int16).pin_memory()
    dev_in = [host_in.cuda() for _ in range(pairs)]
    dev_out = [torch.empty(n, dtype=torch.int16, device="cuda") for _ in range(pairs)]
    ws = hb.DeviceWorkspace(be, 2 * pairs)
    for i in range(pairs):
        ws.bind(2 * i, dev_in[i].data_ptr(), n * 2)
        ws.bind(2 * i + 1, dev_out[i].data_ptr(), n * 2)
    calls = [kc.KernelCall.Gelu(kc.UnaryCall(kc.rb(2 * i), kc.rb(2 * i + 1), n, 16, kc.DTYPE_BF16)) for i in range(pairs)]
    hws = hb.HostWorkspace([host_in.numpy(), host_out.numpy()])
    hcall = kc.KernelCall.Gelu(kc.UnaryCall(kc.rb(0), kc.rb(1), n, 16, kc.DTYPE_BF16))

    def cpu_baseline():
        from oracle import oracle as orc
        x = host_in.numpy().view(np.uint16)
        fast = orc.fast_lib()
        orc.unary_lut(kc.LUT_GELU, kc.DTYPE_BF16, x[:1024], which=fast)
        best = 1e9
        t_end = time.time() + 10
        while time.time() < t_end:
            t0 = time.perf_counter()
            orc.unary_lut(kc.LUT_GELU, kc.DTYPE_BF16, x, which=fast)
            best = min(best, time.perf_counter() - t0)
        return {"value": n * 4 / best / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                "sample": "full 16,777,216-element tensor, best of ~10 s of serial passes (the reference loop is serial)"}

    def ref_step():
        from oracle import oracle as orc
        orc.unary_lut(kc.LUT_GELU, kc.DTYPE_BF16, host_in.numpy().view(np.uint16), which=orc.fast_lib(), mt=True)

    return {
        "name": "lut_gelu_bf16_16777216",
        "metric": "lut_activation_GBps", "unit": "GB/s", "dtype": "u16", "scaling": "weak",
        "run_device": lambda step: be.dispatch(calls[step % pairs], ws),
        "run_host": lambda step: be.dispatch(hcall, hws),
        "ref_step": ref_step, "ref_fraction": 1.0,
        "units_per_step": n * 4 / 1e9,  # GB of algorithmic traffic per step
        "launches_per_step": 1,
        "roofline": {"bound": "hbm", "bytes_per_launch": n * 4, "kernel": "lut_stream_kernel",
                     "traffic": 34_007_808, "traffic_note": "ncu, profiles/lut_stream_kernel_gelu_bf16_16Mi.md: 33.70 MB read + 0.31 MB written inside the kernel window (the output is still dirty in L2)"},
        "h2d": n * 2, "d2h": n * 2,
        "cpu_baseline": cpu_baseline,
        "config": {"workload": LUT_WORKLOAD, "l2": "8 rotated buffer pairs (512 MiB) > 126 MB L2"},
        "keep": (dev_in, dev_out, host_in, host_out),
    }


def workload_attention(be, torch, rank, args, world=1):
    import hologram_b200 as hb
    from hologram_b200 import kernel_call as kc
    b, h, kv, past, d = 32, 32 // world, 8 // world, 8192, 128   # sharded by KV head
    rng = np.random.default_rng(0xC4 + rank)
    rows = b * kv * past

    def quant_on_device(nrows, seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        src = torch.randn(nrows * d, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        codes = torch.empty(nrows * d, dtype=torch.int8, device="cuda")
        scales = torch.empty(nrows, dtype=torch.float32, device="cuda")
        w = hb.DeviceWorkspace(be, 3)
        w.bind(0, src.data_ptr(), nrows * d * 2)
        w.bind(1, codes.data_ptr(), nrows * d)
        w.bind(2, scales.data_ptr(), nrows * 4)
        be.dispatch(kc.KernelCall.QuantizeRowsI8(kc.QuantizeRowsI8Call(kc.rb(0), kc.rb(1), kc.rb(2), nrows, d, kc.DTYPE_BF16)), w)
        be.synchronize()
        return codes, scales

    kp, kps = quant_on_device(rows, 1 + rank)
    vp, vps = quant_on_device(rows, 2 + rank)
    kn, kns = quant_on_device(b * kv, 3 + rank)
    vn, vns = quant_on_device(b * kv, 4 + rank)
    q = torch.from_numpy(bf16_rne(rng.standard_normal(b * h * d).astype(np.float32)).view(np.int16)).cuda()
    vl = torch.tensor([past], dtype=torch.int32, device="cuda")
    out = torch.empty(b * h * d, dtype=torch.int16, device="cuda")
    tensors = [q, kp, kps, vp, vps, kn, kns, vn, vns, vl, out]
    ws = hb.DeviceWorkspace(be, 11)
    for i, t in enumerate(tensors):
        ws.bind(i, t.data_ptr(), t.numel() * t.element_size())
    call = kc.KernelCall.DecodeAttentionValidQ8(kc.DecodeAttentionValidQ8Call(*[kc.rb(i) for i in range(11)], b, h, kv, 1, past, 1, d, 0, kc.DTYPE_BF16))
    host = [t.cpu().pin_memory() for t in tensors]
    hws = hb.HostWorkspace([t.numpy() for t in host])
    algo = 2 * rows * d + 2 * rows * 4 + 2 * b * h * d * 2 + 2 * b * kv * (d + 4)

    def cpu_args(nb):
        f = lambda t, n: t.numpy()[:n]
        hq = host[0].numpy().view(np.uint16)[:nb * h * d]
        return (hq, kc.DTYPE_BF16, f(host[1], nb * kv * past * d), f(host[2], nb * kv * past), f(host[3], nb * kv * past * d),
                f(host[4], nb * kv * past), f(host[5], nb * kv * d), f(host[6], nb * kv), f(host[7], nb * kv * d), f(host[8], nb * kv),
                past, nb, h, kv, 1, past, 1, d, 0)

    def cpu_baseline():
        from oracle import oracle as orc
        nb = 2
        a = cpu_args(nb)
        t0 = time.perf_counter()
        orc.decode_attention_valid_q8(*a, which=orc.fast_lib())
        dt = time.perf_counter() - t0
        return {"value": algo * nb / b / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                "sample": f"{nb} of {b} sequences (dequantize + f32 attention, rows split over all host threads)"}

    def ref_step():
        from oracle import oracle as orc
        orc.decode_attention_valid_q8(*cpu_args(2), which=orc.fast_lib())

    return {
        "name": f"decode_attention_q8_b{b}_h{h}_kv{kv}_d{d}_L{past}",
        "metric": "q8kv_decode_attention_GBps", "unit": "GB/s", "dtype": "i8/f32", "scaling": "strong",
        "run_device": lambda step: be.dispatch(call, ws),
        "run_host": lambda step: be.dispatch(call, hws),
        "ref_step": ref_step, "ref_fraction": 2 / b,
        "units_per_step": algo / 1e9,
        "launches_per_step": 1,
        "roofline": {"bound": "hbm", "bytes_per_launch": algo, "kernel": "decode_attention_q8_kernel",
                     "traffic": 556_297_984 // world, "traffic_note": "ncu at N=1 of the same number of key rows (the decoder's call), profiles/decode_attention_q8_kernel_b32_h32_kv8_L8192.md: 554.48 MB read + 1.81 MB written; divided by N for a shard (traffic is proportional to the rows)"},
        "h2d": sum(t.numel() * t.element_size() for t in tensors[:-1]), "d2h": out.numel() * 2,
        "cpu_baseline": cpu_baseline,
        "config": {"workload": attention_workload_string(b, h * world, kv * world, d, past), "parallelism": f"kv-head shards x{world}",
                   "l2": "KV codes (512 MiB per GPU at N=1) exceed the 126 MB L2"},
        "keep": (tensors, host),
    }


def decoder_workload_string(cfg):
    """The workload description both arms print (the driver compares the two strings)."""
    return (f"config[4]: {cfg.n_layers}-layer Llama-style decoder .holo, d_model {cfg.d_model}, {cfg.n_heads} q / {cfg.n_kv_heads} kv heads, "
            f"head_dim {cfg.head_dim}, SwiGLU {cfg.ffn}, vocab {cfg.vocab}, batch {cfg.batch} x 1 token per step, {cfg.bucket} cached positions, int8 KV")


LUT_WORKLOAD = "config[0]: bf16 GELU via the 65536-entry u16 LUT, 16,777,216 elements, 99% N(0,9) + 1% specials"


def attention_workload_string(b, h, kv, d, past):
    return f"config[3]: single-token decode attention, batch {b}, {h} q / {kv} kv heads, head_dim {d}, {past} cached positions, int8 KV"


def workload_decoder(be, torch, rank, args, world=1):
    """Config 5: 8-layer Llama-style decoder `.holo`, batch 64, 4096 cached positions, int8 KV."""
    import hologram_b200 as hb
    from hologram_b200 import decoder_holo as dh
    from hologram_b200 import kernel_call as kc
    cfg = dh.DecoderConfig()
    if os.environ.get("HOLO_BENCH_LAYERS"):
        cfg.n_layers = int(os.environ["HOLO_BENCH_LAYERS"])
    shapes = {"wq": (cfg.d_model, cfg.n_heads * cfg.head_dim), "wk": (cfg.d_model, cfg.n_kv_heads * cfg.head_dim),
              "wv": (cfg.d_model, cfg.n_kv_heads * cfg.head_dim), "wo": (cfg.n_heads * cfg.head_dim, cfg.d_model),
              "wg": (cfg.d_model, cfg.ffn), "wu": (cfg.d_model, cfg.ffn), "wd": (cfg.ffn, cfg.d_model),
              "embed": (cfg.vocab, cfg.d_model), "lm_head": (cfg.d_model, cfg.vocab)}

    def weights(name):
        # random-init N(0, 0.02^2) bf16, generated on the GPU (same seed on every rank), read back
        base = name.split(".")[-1]
        g = torch.Generator(device="cuda").manual_seed(0xC5 * 1000003 + sum(ord(c) * (i + 1) for i, c in enumerate(name)))
        if base in ("g1", "g2", "gf"):
            t = 1.0 + 0.02 * torch.randn(cfg.d_model, generator=g, device="cuda")
        else:
            t = 0.02 * torch.randn(shapes[base], generator=g, device="cuda")
        return t.to(torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)

    t0 = time.time()
    img, info = dh.build_decoder_step(cfg, rank, world, weights=weights)
    t1 = time.time()
    sess = hb.InferenceSession(be, img, verify=True)
    t2 = time.time()
    nbytes_img = len(img)
    del img
    H, KV, hd, B, L = info["heads"], info["kv_heads"], cfg.head_dim, cfg.batch, cfg.bucket
    # KV cache content: the row quantizer applied on the device to seeded N(0,1) bf16 rows
    rows = B * KV * L
    scratch = hb.DeviceWorkspace(be, 3)
    g = torch.Generator(device="cuda").manual_seed(0xC5 + rank)
    for l in range(cfg.n_layers):
        for which in ("k", "v"):
            src = torch.randn(rows * hd, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
            scratch.bind(0, src.data_ptr(), rows * hd * 2)
            scratch.bind(1, *sess.device_ptr(f"l{l}.{which}_codes"))
            scratch.bind(2, *sess.device_ptr(f"l{l}.{which}_scales"))
            be.dispatch(kc.KernelCall.QuantizeRowsI8(kc.QuantizeRowsI8Call(kc.rb(0), kc.rb(1), kc.rb(2), rows, hd, kc.DTYPE_BF16)), scratch)
            be.synchronize()
            del src
    rng = np.random.default_rng(0xC5)
    position = 4096 + 17
    host = {"token_ids": rng.integers(0, cfg.vocab, size=B).astype(np.int32),
            "pos": np.array([position], dtype=np.int32), "valid_len": np.array([L], dtype=np.int32)}
    host["cos_q"], host["sin_q"] = dh.rope_tables(cfg, position, H)
    host["cos_k"], host["sin_k"] = dh.rope_tables(cfg, position, KV)
    pinned = {k: torch.from_numpy(np.ascontiguousarray(v).view(np.uint8).copy()).pin_memory() for k, v in host.items()}
    for k, v in pinned.items():
        sess.write(k, v.numpy())
    sess.execute()          # eager walk: allocates scratch, builds LUT tables
    be.synchronize()
    use_graph = os.environ.get("HOLO_BENCH_GRAPH", "1") != "0"
    if use_graph:
        sess.capture()
    logits_host = torch.empty(B * info["vocab"], dtype=torch.int16).pin_memory()
    lp, lbytes = sess.device_ptr("logits")
    import ctypes
    from hologram_b200.backend import lib, _check

    def run_host(step):
        for k, v in pinned.items():
            sess.write(k, v.numpy())
        sess.execute()
        _check(lib.holo_b200_workspace_download(sess.workspace._h, kc.rb(sess.port("logits").slot), ctypes.c_void_p(logits_host.data_ptr()), B * info["vocab"] * 2))

    # the dominant kernel of the step (47 % of the ncu launch list): one layer's int8-KV attention
    attn_calls = [sess.call(i) for i in range(sess.n_calls) if sess.call(i).kind == kc.K_DECODE_ATTENTION_VALID_Q8]
    attn_bytes = 2 * rows * (hd + 4) + 2 * B * H * hd * 2 + 2 * B * KV * (hd + 4)

    def run_dominant(step):
        be.dispatch(attn_calls[step % len(attn_calls)], sess.workspace)

    weight_bytes = sum(len(b) for s_, (dt, b) in info["constants"].items()) - cfg.vocab * cfg.d_model * 2 + B * cfg.d_model * 2
    kv_bytes = cfg.n_layers * 2 * rows * (hd + 4)
    algo = weight_bytes + kv_bytes

    def cpu_baseline():
        return decoder_cpu_sample(cfg)

    return {
        "name": f"llama8L_d{cfg.d_model}_b{B}_L{L}_tp{world}",
        "metric": "decode_tokens_per_s", "unit": "tokens/s", "dtype": "bf16 (int8 KV cache, f32 accumulation)", "scaling": "strong",
        "run_device": lambda step: sess.execute(),
        "run_host": run_host,
        "units_per_step": B / world,   # the batch is replicated over the TP group: count it once
        "launches_per_step": sess.n_calls,
        "roofline": {"bound": "hbm", "bytes_per_launch": attn_bytes, "kernel": "decode_attention_q8_kernel, one layer",
                     "run": run_dominant, "traffic": (556_297_984 // world) if (B, L) == (64, 4096) else None,
                     "traffic_note": "ncu capture of this very call in a one-layer archive at N=1 (554.48 MB read + 1.81 MB written), "
                                     "profiles/decode_attention_q8_kernel_b32_h32_kv8_L8192.md; divided by N for a shard (traffic is proportional to the rows)",
                     "step_bytes": algo},
        "h2d": sum(v.numel() for v in pinned.values()), "d2h": B * info["vocab"] * 2,
        "cpu_baseline": cpu_baseline,
        "config": {"workload": decoder_workload_string(cfg), "parallelism": f"tp{world}",
                   "l2": "per-step working set (weights + KV, >= 1 GB per GPU) exceeds the 126 MB L2",
                   "cuda_graph": use_graph, "calls_per_step": sess.n_calls, "fused_pairs": sess.fused_count,
                   "archive_bytes": nbytes_img, "build_s": round(t1 - t0, 1), "load_s": round(t2 - t1, 1),
                   "roofline_note": "roofline = the dominant kernel (one layer's attention) timed alone with CUDA events after the step loop; step_roofline = the whole step"},
        "keep": (sess, pinned, logits_host, scratch),
    }


class DecoderCpuSample:
    """Reference CPU path for the decoder on a bounded sample: one full-shape layer (embedding gather, the layer,
    the final norm and the trailing KV appends) per step through the CPU interpreter on all host threads; the LM
    head product is timed once. tokens/s is extrapolated to the configured layer count."""

    def __init__(self, cfg):
        from hologram_b200 import decoder_holo as dh
        self.cfg = cfg
        one = dh.DecoderConfig(d_model=cfg.d_model, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, head_dim=cfg.head_dim, ffn=cfg.ffn,
                               vocab=cfg.vocab, n_layers=1, batch=cfg.batch, bucket=cfg.bucket)
        rng = np.random.default_rng(5)

        def weights(name):
            base = name.split(".")[-1]
            shp = {"wq": (one.d_model, one.n_heads * one.head_dim), "wk": (one.d_model, one.n_kv_heads * one.head_dim),
                   "wv": (one.d_model, one.n_kv_heads * one.head_dim), "wo": (one.n_heads * one.head_dim, one.d_model),
                   "wg": (one.d_model, one.ffn), "wu": (one.d_model, one.ffn), "wd": (one.ffn, one.d_model),
                   "embed": (one.vocab, one.d_model), "lm_head": (one.d_model, one.vocab)}.get(base, (one.d_model,))
            n = int(np.prod(shp))
            # uniform bf16 bit patterns in the N(0, 0.02^2) magnitude range: content does not change CPU time
            return (rng.integers(0x3A00, 0x3D00, size=n, dtype=np.uint16) | (rng.integers(0, 2, size=n, dtype=np.uint16) << 15)).reshape(shp)

        _, info = dh.build_decoder_step(one, 0, 1, weights=weights)
        slots = {s: np.frombuffer(bytes(body), dtype=np.uint8).copy() for s, (dt, body) in info["constants"].items()}
        for p in info["inputs"]:
            nb = info["slot_bytes"][p.slot]
            if "codes" in p.name:
                slots[p.slot] = rng.integers(-127, 128, size=nb, dtype=np.int8).view(np.uint8)
            elif "scales" in p.name:
                slots[p.slot] = (rng.random(nb // 4, dtype=np.float32) * 0.03).view(np.uint8)
            elif p.name == "valid_len":
                slots[p.slot] = np.array([one.bucket], dtype=np.int32).view(np.uint8)
            elif p.name == "token_ids":
                slots[p.slot] = rng.integers(0, one.vocab, size=one.batch).astype(np.int32).view(np.uint8)
            elif p.name.startswith("cos"):
                slots[p.slot] = np.full(nb // 2, 0x3F80, dtype=np.uint16).view(np.uint8)
            else:
                slots[p.slot] = np.zeros(nb, dtype=np.uint8)
        self.slots = slots
        lm = [c for c in info["calls"] if c.kind == 46][-1]
        self.layer_calls = [c for c in info["calls"] if c is not lm]
        self.lm = lm
        from oracle import interp
        self.interp = interp
        self.layer_step()                          # warm: page the weights in, produce the head's input
        t0 = time.perf_counter()
        interp.run([lm], slots)
        self.t_head = time.perf_counter() - t0

    def layer_step(self):
        t0 = time.perf_counter()
        self.interp.run(self.layer_calls, self.slots)
        return time.perf_counter() - t0

    def t_step(self, t_layer):
        return self.cfg.n_layers * t_layer + self.t_head


def decoder_cpu_sample(cfg):
    s = DecoderCpuSample(cfg)
    t_layer = min(s.layer_step() for _ in range(2))
    t_step = s.t_step(t_layer)
    return {"value": cfg.batch / t_step, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"1 of {cfg.n_layers} layers + LM head at full shapes through the CPU interpreter "
                      f"(layer {t_layer:.2f} s, head {s.t_head:.2f} s), extrapolated to {cfg.n_layers} layers",
            "extrapolated_from_layers": 1, "t_step_s": t_step}


def workload_matmul(be, torch, rank, args, skinny=False):
    """Config 2: bf16 matmul, f32 accumulation, bf16 output. 4096^3 (tensor-core bound) or
    16 x 4096 x 14336 (HBM bound); operands rotated over buffers larger than L2."""
    import hologram_b200 as hb
    from hologram_b200 import kernel_call as kc
    m, k, n = (16, 4096, 14336) if skinny else (4096, 4096, 4096)
    if os.environ.get("HOLO_BENCH_MKN"):
        m, k, n = (int(v) for v in os.environ["HOLO_BENCH_MKN"].split(","))
    sets = max(2, int(300e6 // (2 * (m * k + k * n + m * n))) + 1)
    g = torch.Generator(device="cuda").manual_seed(0xC3 + rank)
    A = [(torch.randn(m * k, generator=g, device="cuda") / k ** 0.5).to(torch.bfloat16) for _ in range(sets)]
    Bm = [(torch.randn(k * n, generator=g, device="cuda") / k ** 0.5).to(torch.bfloat16) for _ in range(sets)]
    C = [torch.empty(m * n, dtype=torch.bfloat16, device="cuda") for _ in range(sets)]
    ws = hb.DeviceWorkspace(be, 3 * sets)
    calls = []
    for i in range(sets):
        for j, t in enumerate((A[i], Bm[i], C[i])):
            ws.bind(3 * i + j, t.data_ptr(), t.numel() * 2)
        calls.append(kc.KernelCall.MatMul(kc.MatMulCall(kc.rb(3 * i), kc.rb(3 * i + 1), kc.rb(3 * i + 2), m, k, n, kc.DTYPE_BF16, 0)))
    host = [t.cpu().pin_memory() for t in (A[0], Bm[0], C[0])]
    hws = hb.HostWorkspace([t.view(torch.int16).numpy() for t in host])
    hcall = kc.KernelCall.MatMul(kc.MatMulCall(kc.rb(0), kc.rb(1), kc.rb(2), m, k, n, kc.DTYPE_BF16, 0))
    flops, nbytes = 2.0 * m * k * n, 2.0 * (m * k + k * n + m * n)

    def cpu_baseline():
        from oracle import oracle as orc
        mm = min(m, 64)
        a = host[0].view(torch.int16).numpy().view(np.uint16)[:mm * k]
        b = host[1].view(torch.int16).numpy().view(np.uint16)
        t0 = time.perf_counter()
        orc.matmul(a, b, mm, k, n, kc.DTYPE_BF16, which=orc.fast_lib())
        dt = time.perf_counter() - t0
        v = (2.0 * mm * k * n / dt / 1e12) if not skinny else (nbytes * mm / m / dt / 1e9)
        return {"value": v, "unit": "TFLOP/s" if not skinny else "GB/s", "cores": os.cpu_count(), "kind": "port",
                "sample": f"{mm} of {m} rows of A against the full B, all host threads"}

    def burst():
        """The kernel timed alone, as the burst peak it is compared with was (best of 10 single launches, the GPU idle
        between them): the back-to-back loop above runs into the power cap within milliseconds, as cuBLAS does too."""
        if skinny:
            return {}
        stream = torch.cuda.current_stream()
        torch.cuda.synchronize()
        time.sleep(1.0)                       # let the power-cap window recover, then ten launches, each timed by itself
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
        be.dispatch(calls[0], ws)             # clocks up
        for i, (e0, e1) in enumerate(evs):
            e0.record(stream)
            be.dispatch(calls[i % sets], ws)
            e1.record(stream)
        torch.cuda.synchronize()
        best = min(e0.elapsed_time(e1) for e0, e1 in evs)
        peaks = measured_peaks()
        tf = flops / (best / 1e3) / 1e12
        return {"burst": {"kernel_us": best * 1e3, "TFLOPs": tf, "frac_of_burst_peak": tf / peaks["bf16_tflops"],
                          "how": "best of 10 launches, each timed by itself, right after a second of idle (before the power cap bites: how the cuBLAS burst peak was taken)"}}

    return {
        "name": f"matmul_bf16_{m}x{k}x{n}",
        "metric": "matmul_bf16_GBps" if skinny else "matmul_bf16_TFLOPs", "unit": "GB/s" if skinny else "TFLOP/s",
        "dtype": "bf16 (f32 accumulation)", "scaling": "weak",
        "run_device": lambda step: be.dispatch(calls[step % sets], ws),
        "run_host": lambda step: be.dispatch(hcall, hws),
        "units_per_step": nbytes / 1e9 if skinny else flops / 1e12,
        "launches_per_step": 1,
        "roofline": ({"bound": "hbm", "bytes_per_launch": nbytes, "kernel": "matmul_bf16_umma_kernel", "traffic": None} if skinny else
                     {"bound": "tensor", "flops_per_launch": flops, "kernel": "matmul_umma_pair_kernel" if (m >= 256 and n >= 256 and -(-m // 256) * -(-n // 256) >= 74) else "matmul_bf16_umma_kernel",
                      "traffic": 82_627_072 if (m, k, n) == (4096, 4096, 4096) else None,
                      "traffic_note": "ncu, profiles/matmul_bf16_umma_kernel.md: 69.58 MB read + 13.05 MB written inside the kernel window"}),
        "h2d": 2 * (m * k + k * n), "d2h": 2 * m * n,
        "cpu_baseline": cpu_baseline, "extra": burst,
        "config": {"workload": f"config[2]: bf16 matmul M={m} K={k} N={n}, f32 accumulation, bf16 output, A,B ~ N(0, 1/K)",
                   "l2": f"{sets} rotated operand sets (> 126 MB L2)"},
        "keep": (A, Bm, C, host),
    }


def workload_w8a8(be, torch, rank, args):
    """Output-major W8A8 decode product (MatMulDequant, wire 116): f32 activations [m, k], int8 weight
    [n, k], per-channel scales; HBM-bound on the weight. Default 1 x 4096 x 14336."""
    import hologram_b200 as hb
    from hologram_b200 import kernel_call as kc
    m, k, n = 1, 4096, 14336
    if os.environ.get("HOLO_BENCH_MKN"):
        m, k, n = (int(v) for v in os.environ["HOLO_BENCH_MKN"].split(","))
    i4 = bool(os.environ.get("HOLO_BENCH_I4"))          # the packed-nibble weight tier (W4A8): half the weight bytes
    e8 = bool(os.environ.get("HOLO_BENCH_E8"))          # the E8 codebook tier (W1A8): one index byte per eight weights
    wbytes = n * k // 8 if e8 else n * k // 2 if i4 else n * k
    qd = kc.DTYPE_E8CB if e8 else kc.DTYPE_I4 if i4 else kc.DTYPE_I8
    sets = max(2, int(300e6 // wbytes) + 1)
    g = torch.Generator(device="cuda").manual_seed(0xC6 + rank)
    A = [torch.randn(m * k, generator=g, device="cuda") for _ in range(sets)]
    W = [torch.randint(0, 256, (wbytes,), generator=g, device="cuda", dtype=torch.uint8) if (i4 or e8) else
         torch.randint(-127, 128, (n * k,), generator=g, device="cuda", dtype=torch.int8) for _ in range(sets)]
    S = [torch.rand(n, generator=g, device="cuda") * 0.02 + 0.001 for _ in range(sets)]
    Z = torch.zeros(n, dtype=torch.int32, device="cuda")
    O = [torch.empty(m * n, device="cuda") for _ in range(sets)]
    CB = torch.randint(-127, 128, (2048,), generator=g, device="cuda", dtype=torch.int8)
    ws = hb.DeviceWorkspace(be, 4 * sets + 2)
    ws.bind(4 * sets, Z.data_ptr(), n * 4)
    ws.bind(4 * sets + 1, CB.data_ptr(), 2048)
    calls = []
    for i in range(sets):
        for j, t in enumerate((A[i], W[i], S[i], O[i])):
            ws.bind(4 * i + j, t.data_ptr(), t.numel() * t.element_size())
        mc = kc.MatMulDequantCall(kc.rb(4 * i), kc.rb(4 * i + 1), kc.rb(4 * i + 2), kc.rb(4 * sets), kc.rb(4 * i + 3), m, k, n, n, 1, qd,
                                  kc.DTYPE_F32, 0, 0, 1, 1, 0, kc.NONE)
        if e8:
            mc.codebook = kc.rb(4 * sets + 1)
        calls.append(kc.KernelCall.MatMulDequant(mc))
    host = [t.cpu().pin_memory() for t in (A[0], W[0], S[0], Z, O[0], CB)]
    hws = hb.HostWorkspace([t.numpy().view(np.uint8) for t in host])
    hc = kc.MatMulDequantCall(kc.rb(0), kc.rb(1), kc.rb(2), kc.rb(3), kc.rb(4), m, k, n, n, 1, qd, kc.DTYPE_F32, 0, 0, 1, 1, 0, kc.NONE)
    if e8:
        hc.codebook = kc.rb(5)
    hcall = kc.KernelCall.MatMulDequant(hc)
    nbytes = float(wbytes + 4 * (m * k + n + m * n))

    def cpu_baseline():
        from oracle import oracle as orc
        a, w, sc = host[0].numpy(), host[1].numpy(), host[2].numpy()
        best, t_end = 1e9, time.time() + 8
        while time.time() < t_end:
            t0 = time.perf_counter()
            orc.matmul_w8a8_omajor(a, w, sc, m, k, n, i4=i4, codebook=host[5].numpy() if e8 else None)
            best = min(best, time.perf_counter() - t0)
        return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                "sample": "the full product, best of ~8 s of serial passes of the scalar restatement"}

    return {
        "name": f"matmul_{'w1a8_e8cb' if e8 else 'w4a8' if i4 else 'w8a8'}_omajor_{m}x{k}x{n}",
        "metric": "matmul_w8a8_GBps", "unit": "GB/s", "dtype": "i4 x i8 -> i32, f32 writeback" if i4 else "i8 x i8 -> i32, f32 writeback", "scaling": "weak",
        "run_device": lambda step: be.dispatch(calls[step % sets], ws),
        "run_host": lambda step: be.dispatch(hcall, hws),
        "units_per_step": nbytes / 1e9, "launches_per_step": 1,
        "roofline": {"bound": "hbm", "bytes_per_launch": nbytes, "kernel": "matmul_e8cb_omajor_kernel" if e8 else "matmul_w8a8_stream_kernel", "traffic": None},
        "h2d": wbytes + 4 * (m * k + 2 * n), "d2h": 4 * m * n,
        "cpu_baseline": cpu_baseline,
        "config": {"workload": f"output-major W8A8 decode product M={m} K={k} N={n} (quantized-weight GEMV, exact integer)",
                   "l2": f"{sets} rotated operand sets (> 126 MB L2)"},
        "keep": (A, W, S, Z, O, host),
    }


def workload_lut_sweep(be, torch, rank, args):
    """config[1]: SiLU, Sigmoid, Tanh, Exp, Erf x {f16, bf16} over [8192, 14336]; one step = the ten cells."""
    import hologram_b200 as hb
    from hologram_b200 import kernel_call as kc
    rows, cols = 8192, 14336
    n = rows * cols
    g = torch.Generator(device="cuda")
    g.manual_seed(0xC2 + rank)
    x = torch.randn(n, device="cuda", generator=g, dtype=torch.float32) * 4.0
    x_bf16 = x.to(torch.bfloat16).view(torch.int16)
    x_f16 = x.to(torch.float16).view(torch.int16)
    x_f16_exp = x.clamp(-20.0, 11.0).to(torch.float16).view(torch.int16)
    del x
    outs = [torch.empty(n, dtype=torch.int16, device="cuda") for _ in range(2)]
    bufs = [x_bf16, x_f16, x_f16_exp] + outs
    ws = hb.DeviceWorkspace(be, len(bufs))
    for i, b in enumerate(bufs):
        ws.bind(i, b.data_ptr(), n * 2)
    acts = [("silu", kc.KernelCall.Silu), ("sigmoid", kc.KernelCall.Sigmoid), ("tanh", kc.KernelCall.Tanh),
            ("exp", kc.KernelCall.Exp), ("erf", kc.KernelCall.Erf)]
    cells = []
    for name, ctor in acts:
        for dt, dname in ((kc.DTYPE_F16, "f16"), (kc.DTYPE_BF16, "bf16")):
            src = 0 if dt == kc.DTYPE_BF16 else (2 if name == "exp" else 1)
            cells.append((f"{name}_{dname}", ctor(kc.UnaryCall(kc.rb(src), kc.rb(3 + len(cells) % 2), n, 16, dt))))

    def run_device(step):
        for _, call in cells:
            be.dispatch(call, ws)

    sample = 16_777_216
    host_in = x_bf16[:sample].cpu().pin_memory()
    host_out = torch.empty(sample, dtype=torch.int16).pin_memory()
    hws = hb.HostWorkspace([host_in.numpy(), host_out.numpy()])
    hcall = kc.KernelCall.Silu(kc.UnaryCall(kc.rb(0), kc.rb(1), sample, 16, kc.DTYPE_BF16))

    def per_cell():
        stream = torch.cuda.current_stream()
        res = {}
        for name, call in cells:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            be.dispatch(call, ws)
            e0.record(stream)
            for _ in range(5):
                be.dispatch(call, ws)
            e1.record(stream)
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 5 * 1e3
            res[name] = {"us": round(us, 2), "GBps": round(n * 4 / us / 1e3, 1)}
        return {"cells": res}

    def cpu_baseline():
        from oracle import oracle as orc
        xs = host_in.numpy().view(np.uint16)
        fast = orc.fast_lib()
        orc.unary_lut(kc.LUT_SILU, kc.DTYPE_BF16, xs[:1024], which=fast)
        best, t_end = 1e9, time.time() + 10
        while time.time() < t_end:
            t0 = time.perf_counter()
            orc.unary_lut(kc.LUT_SILU, kc.DTYPE_BF16, xs, which=fast)
            best = min(best, time.perf_counter() - t0)
        return {"value": sample * 4 / best / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                "sample": "SiLU bf16 over the first 16,777,216 elements of the tensor, best of ~10 s of serial passes (the reference loop is serial)"}

    return {
        "name": "lut_sweep_5acts_2dtypes_8192x14336",
        "metric": "lut_activation_GBps", "unit": "GB/s", "dtype": "u16", "scaling": "weak",
        "run_device": run_device,
        "run_host": lambda step: be.dispatch(hcall, hws), "e2e_units_per_step": sample * 4 / 1e9,
        "units_per_step": len(cells) * n * 4 / 1e9,
        "roofline": {"bound": "hbm", "bytes_per_launch": len(cells) * n * 4, "kernel": "lut_stream_kernel (ten launches per step)",
                     "traffic": None, "traffic_note": "not captured at this size; the 16,777,216-element capture shows input read once"},
        "h2d": sample * 2, "d2h": sample * 2,
        "extra": per_cell,
        "cpu_baseline": cpu_baseline,
        "config": {"workload": "config[1]: SiLU/Sigmoid/Tanh/Exp/Erf x f16/bf16 LUT over [8192, 14336], N(0,16) rounded to dtype (Exp f16 clamped to [-20, 11])",
                   "l2": "each cell streams 470 MB > 126 MB L2", "e2e": "one SiLU bf16 call over 16,777,216 elements through host buffers",
                   "exp_erf_tables": "parity unpinned: built from the f64 function rounded to f32 (the reference links libm 0.2.16, absent here); "
                                     "holo_b200_ctx_set_lut_table installs tables produced by the reference itself"},
        "keep": (bufs, host_in, host_out),
    }


WORKLOADS = {"lut": workload_lut, "lut_sweep": workload_lut_sweep, "w8a8": workload_w8a8, "attention": workload_attention, "decoder": workload_decoder,
             "matmul": workload_matmul, "gemv": lambda *a: workload_matmul(*a, skinny=True)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=os.environ.get("HOLO_BENCH_WORKLOAD", "decoder"))
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sub", action="store_true", help="decoder workload: skip the LUT and attention sub-results")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="profiling aid, one GPU: run rank 0's shard of an N-way tensor-parallel attention / decoder without the "
                         "exchange between ranks (the kernels then have the shapes of an N-GPU run); not a benchmark line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    # Libraries loaded below may write to stdout (NCCL prints its version there): stdout carries the one JSON
    # line and nothing else, everything else goes to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        os.write(json_fd, (json.dumps(obj) + "\n").encode())

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        return main_reference(args, rank, world, emit)

    import torch
    import torch.distributed as dist
    import hologram_b200 as hb

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    be = hb.B200Backend(local_rank)
    stream = torch.cuda.Stream()          # a real stream: the legacy default stream cannot be captured into a graph
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)

    if world > 1 and args.workload == "decoder":
        uid = [hb.B200Backend.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        be.init_tp(uid[0], rank, world)
    fn = WORKLOADS[args.workload]
    shard_world = args.shard_of if (args.shard_of > 1 and world == 1) else world
    wl = fn(be, torch, rank, args, shard_world) if args.workload in ("attention", "decoder") else fn(be, torch, rank, args)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(run, steps, warmup):
        for s in range(warmup):
            run(s)
        barrier()
        l0 = be.launch_count
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for s in range(steps):
            run(warmup + s)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        launches = be.launch_count - l0
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches

    def repeats_for(run, steps, warmup):
        """How often the block of `steps` steps is repeated inside one event pair so that the timed region covers
        at least 64 steps and at least ~120 ms (the clock sampler then sees it under load). Agreed over the ranks."""
        est_ms, _ = timed(run, min(steps, 5), warmup)
        per_step = max(est_ms / min(steps, 5), 1e-4)
        reps = max(-(-64 // steps), int(np.ceil(120.0 / (per_step * steps))), 1)
        if world > 1:
            t = torch.tensor([reps], device="cuda", dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            reps = int(t.item())
        return reps

    def measure(w, steps, warmup):
        """One workload: device-resident timing over `steps` x repeats steps with its own clock sample."""
        reps = repeats_for(w["run_device"], steps, warmup)
        try:
            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
        except Exception:
            uuid = None
        smp = ClockSampler(local_rank, uuid)
        if rank == 0:
            smp.start()
        total_ms, n_launch = timed(w["run_device"], steps * reps, 3)
        clk = smp.stop() if rank == 0 else None
        return total_ms / reps, n_launch // reps, reps, clk

    ms, launches, repeats, clocks = measure(wl, args.steps, args.warmup)
    dom_ms = None
    if "run" in wl["roofline"]:
        dom_steps = 24
        dom_total, _ = timed(wl["roofline"]["run"], dom_steps, 3)
        dom_ms = dom_total / dom_steps

    e2e = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 10))
        ems, _ = timed(wl["run_host"], e2e_steps, 2)
        e2e = {"value": wl.get("e2e_units_per_step", wl["units_per_step"]) * world * e2e_steps / (ems / 1e3), "unit": wl["unit"],
               "h2d_bytes_per_step": wl["h2d"], "d2h_bytes_per_step": wl["d2h"], "steps": e2e_steps}

    if rank == 0:
        peaks = measured_peaks()
        per_step_ms = ms / args.steps
        value = wl["units_per_step"] * world * args.steps / (ms / 1e3)
        kernel_ms = dom_ms if dom_ms is not None else per_step_ms
        if wl["roofline"]["bound"] == "tensor":
            achieved = wl["roofline"]["flops_per_launch"] / (kernel_ms / 1e3) / 1e12
            # launches back to back for >= 120 ms run under the power cap: the sustained cuBLAS figure is the like-for-like peak
            peak, punit = peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"], "TFLOP/s"
        else:
            achieved = wl["roofline"]["bytes_per_launch"] / (kernel_ms / 1e3) / 1e9
            peak, punit = peaks["hbm_gbs"], "GB/s"
        line = {
            "metric": wl["metric"], "value": value, "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_step_ms, "timed_steps": args.steps * repeats, "repeats": repeats,
            "higher_is_better": True, "scaling": wl["scaling"],
            "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic (seeded)",
            "config": dict(wl["config"], name=wl["name"]),
            "clocks": clocks, "gpu_launches": launches,
            "roofline": {"bound": wl["roofline"]["bound"], "kernel": wl["roofline"].get("kernel"), "achieved": achieved, "peak": peak,
                         "unit": punit, "frac": achieved / peak, "kernel_us": kernel_ms * 1e3,
                         "traffic": wl["roofline"].get("traffic"), "traffic_note": wl["roofline"].get("traffic_note"),
                         "peak_source": peaks["source"] + (" (MEASURED_PEAKS.json cuBLAS bf16, sustained loop: the timed region is a back-to-back loop under the power cap)"
                                                           if wl["roofline"]["bound"] == "tensor" else " (MEASURED_PEAKS.json copy bandwidth)")},
            "e2e": e2e,
        }
        if wl["roofline"]["bound"] == "tensor":
            line["roofline"]["frac_of_burst_peak"] = achieved / peaks["bf16_tflops"]
        else:
            line["roofline"]["frac_of_nominal_8TBps"] = achieved / 8000.0
        if "step_bytes" in wl["roofline"]:
            sb = wl["roofline"]["step_bytes"] / (per_step_ms / 1e3) / 1e9
            line["step_roofline"] = {"bound": "hbm", "achieved": sb, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": sb / peaks["hbm_gbs"],
                                     "note": "whole step: per-GPU matmul weights + KV codes and scales read once / step time"}
        if "extra" in wl:
            line.update(wl["extra"]())
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = wl["cpu_baseline"]()
    # The rest of the metric (LUT and quantized-KV attention GB/s against the HBM peak) beside the decoder line:
    # config[0] as per-GPU replicas, config[3] sharded by KV head over the same ranks. Every rank takes part.
    sub = {}
    if args.workload == "decoder" and not args.no_sub:
        del wl
        for name in ("lut", "attention"):
            w = WORKLOADS[name](be, torch, rank, args, world) if name == "attention" else WORKLOADS[name](be, torch, rank, args)
            sms, sl, sreps, sclk = measure(w, 16, 5)
            if rank == 0:
                peaks = measured_peaks()
                us = sms / 16 * 1e3
                gbs = w["roofline"]["bytes_per_launch"] / us / 1e3
                sub[name] = {"metric": w["metric"], "workload": w["config"]["workload"], "parallelism": w["config"].get("parallelism", f"replicas x{world}"),
                             "value": w["units_per_step"] * world * 16 / (sms / 1e3), "unit": w["unit"], "kernel": w["roofline"]["kernel"],
                             "kernel_us": us, "per_gpu_GBps": gbs, "frac": gbs / peaks["hbm_gbs"], "frac_of_nominal_8TBps": gbs / 8000.0,
                             "bytes_per_launch": w["roofline"]["bytes_per_launch"], "timed_steps": 16 * sreps, "clocks": sclk, "l2": w["config"]["l2"]}
            del w
            torch.cuda.empty_cache()
    if rank == 0:
        if sub:
            line["sub"] = sub
        if shard_world != world:
            line["profiling_only"] = f"rank 0's shard of a {shard_world}-way run on one GPU, no exchange between ranks"
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def main_reference(args, rank, world, emit):
    """The reference's CPU implementation of the path (the C restatement, all host threads),
    timed on a bounded sample per step. Rank 0 only."""
    if rank != 0:
        return
    import types
    torch = None
    try:
        import torch as _t
        torch = _t
    except Exception:
        pass
    # host-only construction of the same inputs
    from hologram_b200 import kernel_call as kc
    from oracle import oracle as orc
    wlname = args.workload
    if wlname == "decoder":
        from hologram_b200 import decoder_holo as dh
        cfg = dh.DecoderConfig()
        sample = DecoderCpuSample(cfg)             # set-up and the LM head (timed once) stay outside the steps
        for _ in range(args.warmup):
            sample.layer_step()
        t_layers = [sample.layer_step() for _ in range(max(1, args.steps))]
        t_step = sample.t_step(float(np.mean(t_layers)))
        value = cfg.batch / t_step
        emit({
            "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(t_layers), "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 (int8 KV cache, f32 accumulation)", "data": "synthetic (seeded)",
            "config": {"workload": decoder_workload_string(cfg), "parallelism": f"tp{args.gpus}",
                       "note": "the CPU path has no tensor parallelism: the same step on the host cores at every N"},
            "extrapolated_from_layers": 1,
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                             "sample": f"per step: 1 of {cfg.n_layers} layers at full shapes on all host threads (mean {np.mean(t_layers):.2f} s), "
                                       f"the LM head timed once ({sample.t_head:.2f} s); ms_per_step = {cfg.n_layers} x layer + head"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        })
        return
    if wlname == "lut":
        n = 16_777_216
        x = synth_c1(n, 0xC1)
        units = n * 4 / 1e9
        step = lambda: orc.unary_lut(kc.LUT_GELU, kc.DTYPE_BF16, x, which=orc.fast_lib(), mt=True)
        frac, metric, unit, dtype = 1.0, "lut_activation_GBps", "GB/s", "u16"
        cfg = {"workload": LUT_WORKLOAD}
        sample = "full tensor per step, table lookups partitioned over all host threads"
    else:
        b, h, kv, past, d, nb = 32, 32, 8, 8192, 128, 2
        rng = np.random.default_rng(0xC4)
        q = bf16_rne(rng.standard_normal(nb * h * d).astype(np.float32))
        mk = lambda rows: orc.quantize_rows_i8(bf16_rne(rng.standard_normal(rows * d).astype(np.float32)), kc.DTYPE_BF16, rows, d)
        kp, vp, kn, vn = mk(nb * kv * past), mk(nb * kv * past), mk(nb * kv), mk(nb * kv)
        algo = 2 * b * kv * past * (d + 4) + 2 * b * h * d * 2 + 2 * b * kv * (d + 4)
        units = algo / 1e9
        step = lambda: orc.decode_attention_valid_q8(q, kc.DTYPE_BF16, kp[0], kp[1], vp[0], vp[1], kn[0], kn[1], vn[0], vn[1],
                                                     past, nb, h, kv, 1, past, 1, d, 0, which=orc.fast_lib())
        frac, metric, unit, dtype = nb / b, "q8kv_decode_attention_GBps", "GB/s", "i8/f32"
        cfg = {"workload": attention_workload_string(b, h, kv, d, past)}
        sample = f"{nb} of {b} sequences per step"
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = units * frac * args.steps / dt
    cores = os.cpu_count()
    emit({
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3 / frac, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": dtype, "data": "synthetic (seeded)", "config": cfg,
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


if __name__ == "__main__":
    main()
