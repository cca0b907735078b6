"""Tensor-parallel decoder: host-side logic on CPU (gloo, world size 2), GPU runs at N = 2 and N = 4."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
sys.path.insert(0, %(root)r); sys.path.insert(0, os.path.join(%(root)r, "tests"))
import numpy as np, torch, torch.distributed as dist
from hologram_b200 import decoder_holo as dh
from oracle import oracle as orc
from decoder_common import oracle_step, step_inputs, small_cfg
mode = %(mode)r
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
cfg = %(cfg)s
img, info = dh.build_decoder_step(cfg, rank, world)
vals = step_inputs(cfg, info, 9, 128, seed=11, tp_rank=rank)
if mode == "cpu":
    dist.init_process_group("gloo")
    def all_reduce(x):
        t = torch.from_numpy(np.ascontiguousarray(x)); dist.all_reduce(t); return t.numpy()
    slots = oracle_step(info, vals, all_reduce=all_reduce)
    logits = orc.bf16_to_f32(slots[info["outputs"][0].slot].view(np.uint16))
else:
    import hologram_b200 as hb
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo")
    be = hb.B200Backend(rank)
    uid = [hb.B200Backend.nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    be.init_tp(uid[0], rank, world)
    # a bare AllReduce through the C ABI: 64 x 4096 bf16 partials, seeded per rank, twice in a
    # row (the second call reuses the other message slot and the next epoch)
    from hologram_b200 import kernel_call as kc
    n = 64 * 4096
    ws = hb.DeviceWorkspace(be, 1)
    for rep in range(3):
        part = orc.f32_to_bf16_rne(np.random.default_rng(100 * rep + rank).standard_normal(n).astype(np.float32))
        ws.put(0, part)
        be.dispatch(kc.KernelCall.AllReduce(kc.AllReduceCall(kc.rb(0), n, kc.DTYPE_BF16)), ws)
        np.save(os.path.join(%(out)r, f"allreduce_{rep}_{rank}.npy"), ws.read(0, dtype=np.uint16).copy())
    ws.close()
    with open(os.path.join(%(out)r, f"transport_{rank}.txt"), "w") as f:
        f.write(str(be.tp_transport))
    sess = hb.InferenceSession(be, img)
    for name, arr in vals.items():
        sess.write(name, arr)
    sess.execute()
    logits = orc.bf16_to_f32(sess.read("logits", np.uint16))
    sess.close()
    be.close()
np.save(os.path.join(%(out)r, f"logits_{mode}_{rank}.npy"), logits)
dist.destroy_process_group()
'''


SMALL = "small_cfg(layers=1, batch=2, bucket=128)"
# four KV heads, so that four ranks each own one; the row-parallel products take the fused all-reduce epilogue
WIDE = ("dh.DecoderConfig(d_model=1024, n_heads=8, n_kv_heads=4, head_dim=128, ffn=2048, vocab=2048, n_layers=2, "
        "batch=8, bucket=128)")


def _launch(mode, tmp_path, world=2, cfg=SMALL, **extra_env):
    script = tmp_path / f"worker_{mode}.py"
    script.write_text(WORKER % {"root": ROOT, "mode": mode, "out": str(tmp_path), "cfg": cfg})
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra_env)
    port = 29500 + os.getpid() % 500
    subprocess.check_call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)], env=env, timeout=600)
    return [np.load(tmp_path / f"logits_{mode}_{r}.npy") for r in range(world)]


def _single_rank_reference():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from hologram_b200 import decoder_holo as dh
    from oracle import oracle as orc
    from decoder_common import oracle_step, step_inputs, small_cfg
    cfg = small_cfg(layers=1, batch=2, bucket=128)
    _, info = dh.build_decoder_step(cfg, 0, 1)
    # the TP ranks each quantize their own KV heads with per-rank seeds: rebuild the full cache
    _, i0 = dh.build_decoder_step(cfg, 0, 2)
    parts = [step_inputs(cfg, i0, 9, 128, seed=11, tp_rank=r) for r in range(2)]
    vals = step_inputs(cfg, info, 9, 128, seed=11)
    B, L, hd = cfg.batch, cfg.bucket, cfg.head_dim
    for name in list(vals):
        if "codes" in name or "scales" in name:
            w = hd if "codes" in name else 1
            a, b = (p[name].reshape(B, 1, L, w) for p in parts)
            vals[name] = np.ascontiguousarray(np.concatenate([a, b], axis=1)).reshape(-1)
    slots = oracle_step(info, vals)
    return orc.bf16_to_f32(slots[info["outputs"][0].slot].view(np.uint16)).reshape(B, cfg.vocab)


def test_tp2_interpreter_over_gloo_matches_single_rank(tmp_path):
    r0, r1 = _launch("cpu", tmp_path)
    want = _single_rank_reference()
    got = np.concatenate([r0.reshape(want.shape[0], -1), r1.reshape(want.shape[0], -1)], axis=1)
    err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
    assert err <= 2e-2, err


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [False, True])
def test_tp2_on_two_gpus_matches_single_rank(tmp_path, fused):
    # fused: the all-reduce inside the row-parallel product's epilogue (opt-in); otherwise product, then all-reduce kernel
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r0, r1 = _launch("gpu", tmp_path, **({"HOLO_TP_FUSED_GEMM": "1"} if fused else {}))
    # the bare all-reduces: both ranks hold the same bits; over peer memory they are exactly the
    # f32 sum in rank order, truncated to bf16 (NCCL rounds and orders differently: tolerance)
    sys.path.insert(0, ROOT)
    from oracle import oracle as orc
    transport = [int(open(tmp_path / f"transport_{r}.txt").read()) for r in range(2)]
    assert transport[0] == transport[1] and transport[0] in (1, 2)
    for rep in range(3):
        got = [np.load(tmp_path / f"allreduce_{rep}_{r}.npy") for r in range(2)]
        assert np.array_equal(got[0], got[1])
        parts = [orc.bf16_to_f32(orc.f32_to_bf16_rne(np.random.default_rng(100 * rep + r).standard_normal(64 * 4096).astype(np.float32)))
                 for r in range(2)]
        total = (np.float32(0.0) + parts[0]) + parts[1]
        if transport[0] == 2:
            assert np.array_equal(got[0], (total.view(np.uint32) >> 16).astype(np.uint16))
        else:
            assert np.max(np.abs(orc.bf16_to_f32(got[0]) - total)) <= 2.0 ** -6 * np.max(np.abs(total))
    want = _single_rank_reference()
    got = np.concatenate([r0.reshape(want.shape[0], -1), r1.reshape(want.shape[0], -1)], axis=1)
    err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
    assert err <= 2e-2, err


WIDE8 = ("dh.DecoderConfig(d_model=2048, n_heads=16, n_kv_heads=8, head_dim=128, ffn=4096, vocab=4096, n_layers=2, "
         "batch=8, bucket=128)")


def _tp4(tmp_path, world=4, cfg=WIDE, **extra_env):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    want = np.concatenate([r.reshape(8, -1) for r in _launch("cpu", tmp_path, world, cfg)], axis=1)
    got = np.concatenate([r.reshape(8, -1) for r in _launch("gpu", tmp_path, world, cfg, **extra_env)], axis=1)
    for rep in range(3):
        res = [np.load(tmp_path / f"allreduce_{rep}_{r}.npy") for r in range(world)]
        assert all(np.array_equal(res[0], x) for x in res[1:])
    err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
    assert err <= 2e-2, err


@pytest.mark.gpu
def test_tp4_on_four_gpus_matches_the_gloo_interpreter(tmp_path):
    # the same per-rank archives through the CPU interpreter (all-reduce over gloo) and through the
    # sessions on four GPUs (products, then the all-reduce kernel over peer memory)
    _tp4(tmp_path)


@pytest.mark.gpu
def test_tp4_with_the_all_reduce_in_the_product_epilogue(tmp_path):
    # groups above two ranks take the fused product + all-reduce only when asked
    _tp4(tmp_path, HOLO_TP_FUSED_GEMM_ANY_WORLD="1")


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [False, True])
def test_tp8_on_eight_gpus_matches_the_gloo_interpreter(tmp_path, fused):
    _tp4(tmp_path, 8, WIDE8, **({"HOLO_TP_FUSED_GEMM_ANY_WORLD": "1"} if fused else {}))
