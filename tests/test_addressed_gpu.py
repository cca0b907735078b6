"""Content-addressed execution on the device: resident values are bound by pointer instead of
recomputed, whole-graph repeats are answered from the memo, pool bytes stay bounded, leased values
survive and force the honest copy, uniquely owned caches move in place
(crates/hologram-exec/src/session.rs:942-1030, 1052-1289, 1313-1370; crates/hologram-exec/tests/confinement.rs,
crates/hologram-exec/tests/lease.rs)."""
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
    # the schedule the compiler would emit: the x branch one level before the z branch, so the residual of the
    # fused MatMulAdd is ready strictly before the matmul that absorbs it (session.rs:2268-2277)
    w.exec_plan = [[0], [1], [2], [3]]
    return w.finish(), (m, k, n, w1, w2)


def expect(x, z, m, k, n, w1, w2):
    a1 = orc.matmul(x, w1, m, k, n, BF, act=kc.FUSED_SILU)
    return orc.binary(0, a1, orc.matmul(z, w2, m, k, n, BF), BF)


def test_subgraph_reuse_memo_and_bounded_pool(backend):
    img, (m, k, n, w1, w2) = two_branch_archive()
    sess = hb.InferenceSession(backend, img, addressed=True)
    x, z1, z2 = (synth_bf16(m * k, 1.0, s) for s in (10, 11, 12))

    def run(x, z):
        # inputs enter by label: intern_input hashes the bytes once and stores them in the pool (session.rs:1018-1022)
        lx, lz = sess.intern_input(x), sess.intern_input(z)
        assert (lx, lz) == (hs.label_bytes(x), hs.label_bytes(z))
        labels, st = sess.execute_addressed([lx, lz])
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
    # the labels are the derivation of the fused call list: interior values by the cheap derivation, the graph
    # output under the boundary form (address.rs:197-221)
    lx, lz = hs.label_bytes(x), hs.label_bytes(z2)
    lw1, lw2 = hs.label_bytes(w1), hs.label_bytes(w2)
    op, pr = hs.op_signature(sess.call(0))
    a1 = hs.label_derive(op, pr, [lx, lw1])
    op, pr = hs.op_signature(sess.call(1))
    assert l2[0] == hs.label_derive_boundary(op, pr, [lz, lw2, a1])     # operands in kernel order: a, b, residual
    assert np.array_equal(sess.resolve(l2[0], np.uint16), o2) and sess.resolve(a1) is not None
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
    plain.execute()
    # a label that was never interned is refused before anything changes (session.rs:959-971)
    with pytest.raises(hb.BackendError) as e:
        addr.execute_addressed([hs.label_bytes(vals[p.name]) for p in addr.inputs])
    assert e.value.variant == "ShapeMismatch" and "not resident" in str(e.value)
    labels, st = addr.execute_addressed([addr.intern_input(vals[p.name]) for p in addr.inputs])
    # every call ran; the four KvCacheWrite calls as in-place moves of their (uniquely owned) cache buffers
    assert st.memo_hit == 0 and st.dispatched + st.moved == addr.n_calls and st.moved == 4 * cfg.n_layers
    assert np.array_equal(addr.read("logits", np.uint16), plain.read("logits", np.uint16))
    for name in ("l0.k_codes_next", "l0.v_scales_next"):
        assert np.array_equal(addr.read(name), plain.read(name))
    assert all(len(l) == 71 and l.startswith(b"blake3:") for l in labels)
    # the same step again is a memo hit with the same labels and the same logits
    labels2, st2 = addr.execute_addressed([hs.label_bytes(vals[p.name]) for p in addr.inputs])
    assert st2.memo_hit == 1 and labels2 == labels
    assert np.array_equal(addr.read("logits", np.uint16), plain.read("logits", np.uint16))
    # a new position only: the embedding / norm / projections of the same tokens are reused
    # (the caches of the first step were moved into its outputs: their labels are gone, the values are interned again)
    vals2 = dict(vals)
    vals2["pos"] = np.array([101], dtype=np.int32)
    _, st3 = addr.execute_addressed([addr.intern_input(vals2[p.name]) for p in addr.inputs])
    assert st3.memo_hit == 0 and st3.skipped > st3.moved and st3.dispatched + st3.moved < addr.n_calls
    plain.close()
    addr.close()


# ---- leases (crates/hologram-exec/tests/lease.rs) ------------------------------------------------
DIMS = (2, 2, 8, 16)          # batch, kv heads, bucket rows, row floats


def write_archive():
    """KvCacheWrite(cache, new, pos) -> output, every operand an input port (lease.rs write_graph)."""
    b, hkv, bucket, d = DIMS
    w = holo.HoloWriter()
    cache_b, new_b = b * hkv * bucket * d * 4, b * hkv * d * 4
    w.inputs = [holo.Port("cache", 0, cache_b // 4, kc.DTYPE_F32, [b, hkv, bucket, d]), holo.Port("new", 1, new_b // 4, kc.DTYPE_F32, [b, hkv, 1, d]),
                holo.Port("pos", 2, 1, kc.DTYPE_I32, [1])]
    w.outputs = [holo.Port("out", 3, cache_b // 4, kc.DTYPE_F32, [b, hkv, bucket, d])]
    w.calls = [kc.KernelCall.KvCacheWrite(kc.KvCacheWriteCall(kc.rb(0, 0, cache_b), kc.rb(1, 0, new_b), kc.rb(2, 0, 4), kc.rb(3, 0, cache_b),
                                                              b * hkv, bucket, 1, d * 4))]
    return w.finish()


def f32s(n, seed):
    return (((np.arange(n) * 19 + seed * 23) % 47).astype(np.float32) - 23.0) * np.float32(0.031)


def direct_write(cache, new, pos):
    """The honest-copy kernel through the oracle, as the reference test dispatches it directly."""
    b, hkv, bucket, d = DIMS
    rc, out = orc.kv_cache_write(cache.view(np.uint8), new.view(np.uint8), pos, b * hkv, bucket, 1, d * 4)
    assert rc == 0
    return out.view(np.float32)


def test_leased_label_survives_unrelated_walks_and_ages_out_after_release(backend):
    b, hkv, bucket, d = DIMS
    n_cache, n_new = b * hkv * bucket * d, b * hkv * d
    sess = hb.InferenceSession(backend, write_archive(), addressed=True)
    cache = f32s(n_cache, 1)
    parked = sess.intern_input(cache)
    sibling = sess.intern_input(f32s(n_cache, 2))
    assert sess.retain_label(parked) and sess.leased_count == 1
    other = f32s(n_cache, 3)
    lo = sess.intern_input(other)
    for step in range(3):                      # three unrelated walks (an interleaved conversation's steps)
        new = f32s(n_new, 40 + step)
        want = direct_write(other, new, step)
        out, st = sess.execute_addressed([lo, sess.intern_input(new), sess.intern_input(np.array([step], dtype=np.uint32))])
        assert np.array_equal(sess.resolve(out[0], np.float32), want)
        assert (st.moved, st.dispatched) == (1, 0)          # an owned cache moves in place
        lo, other = out[0], want
    assert np.array_equal(sess.resolve(parked, np.float32), cache)        # the lease held ...
    assert sess.resolve(sibling) is None                                  # ... recency did not
    assert sess.release_label(parked)
    new = f32s(n_new, 50)
    out, st = sess.execute_addressed([parked, sess.intern_input(new), sess.intern_input(np.array([1], dtype=np.uint32))])
    assert np.array_equal(sess.resolve(out[0], np.float32), direct_write(cache, new, 1))
    assert sess.resolve(parked) is None and st.moved == 1                 # an unleased value is owned, hence moved
    sess.close()


def test_lease_forces_the_honest_copy_and_release_restores_the_move(backend):
    b, hkv, bucket, d = DIMS
    n_cache, n_new = b * hkv * bucket * d, b * hkv * d
    sess = hb.InferenceSession(backend, write_archive(), addressed=True)
    cache = f32s(n_cache, 1)
    pre = sess.intern_input(cache)
    assert sess.retain_label(pre)
    pos4 = np.array([4], dtype=np.uint32)
    draft = f32s(n_new, 7)                      # speculative step on the borrowed cache
    out, st = sess.execute_addressed([pre, sess.intern_input(draft), sess.intern_input(pos4)])
    assert np.array_equal(sess.resolve(out[0], np.float32), direct_write(cache, draft, 4))
    assert (st.dispatched, st.moved) == (1, 0)                            # a borrowed cache takes the copy
    assert np.array_equal(sess.resolve(pre, np.float32), cache)           # the rollback point is intact
    real = f32s(n_new, 8)                       # reject the draft: step again from the same pre-image
    out2, _ = sess.execute_addressed([pre, sess.intern_input(real), sess.intern_input(pos4)])
    assert np.array_equal(sess.resolve(out2[0], np.float32), direct_write(cache, real, 4))
    assert sess.release_label(pre)              # accept: the next step owns the value and moves
    out3, st3 = sess.execute_addressed([pre, sess.intern_input(f32s(n_new, 9)), sess.intern_input(np.array([5], dtype=np.uint32))])
    assert (st3.dispatched, st3.moved) == (0, 1)
    assert sess.resolve(pre) is None and sess.resolve(out3[0]) is not None
    # leases are refcounted; a label that is not resident cannot be leased
    l = sess.intern_input(f32s(n_cache, 5))
    assert sess.retain_label(l) and sess.retain_label(l) and sess.release_label(l)
    out4, st4 = sess.execute_addressed([l, sess.intern_input(f32s(n_new, 4)), sess.intern_input(np.array([2], dtype=np.uint32))])
    assert st4.dispatched == 1 and sess.resolve(l) is not None
    assert sess.release_label(l) and not sess.release_label(l)
    assert not sess.retain_label(hs.label_bytes(np.array([1, 2, 3, 4], dtype=np.uint8)))
    sess.close()


def test_decode_loop_by_labels_keeps_pool_bytes_constant(backend):
    # the decode loop of the reference: each step's cache outputs are fed back by label (no upload, no copy), the
    # KvCacheWrite calls move in place, and after warm-up the pool allocates nothing more (tests/confinement.rs)
    cfg = small_cfg(layers=1, batch=2, bucket=128)
    img, info = dh.build_decoder_step(cfg)
    plain = hb.InferenceSession(backend, img)
    addr = hb.InferenceSession(backend, img, addressed=True)
    vals = step_inputs(cfg, info, 100, 100, seed=5)
    labels = {p.name: addr.intern_input(vals[p.name]) for p in addr.inputs}
    for name, arr in vals.items():
        plain.write(name, arr)
    sizes = []
    for step in range(9):
        v = step_inputs(cfg, info, 100 + step, 100 + step, seed=5)
        for name in ("pos", "valid_len", "cos_q", "sin_q", "cos_k", "sin_k"):
            plain.write(name, v[name])
        for name in ("token_ids", "pos", "valid_len", "cos_q", "sin_q", "cos_k", "sin_k"):
            labels[name] = addr.intern_input(v[name])     # interning again keeps an unchanged value live (it promotes the label)
        plain.execute()
        outs, st = addr.execute_addressed([labels[p.name] for p in addr.inputs])
        assert st.moved == 4 * cfg.n_layers and st.memo_hit == 0
        assert np.array_equal(addr.read("logits", np.uint16), plain.read("logits", np.uint16))
        for port, lab in zip(addr.outputs, outs):
            if port.name.endswith("_next"):
                labels[port.name[:-5]] = lab          # this step's cache is the next step's input, by label
        sizes.append(st.pool_bytes)
    assert np.array_equal(addr.read("l0.k_codes_next"), plain.read("l0.k_codes_next"))
    assert len(set(sizes[-3:])) == 1, sizes
    plain.close()
    addr.close()


def test_in_place_calls_keep_their_value_under_addressing(backend):
    # MatMul -> AllReduce -> output, loaded addressed at world 1: the all-reduce rewrites the product where it lies,
    # so the slot must keep its binding (not a fresh zero-filled buffer) and the value loses its derived label
    m, k, n = 32, 256, 512
    w = holo.HoloWriter()
    wt = synth_bf16(k * n, 0.05, 7)
    w.add_constant(1, BF, wt.tobytes())
    w.inputs = [holo.Port("x", 0, m * k, BF, [m, k])]
    w.outputs = [holo.Port("y", 2, m * n, BF, [m, n])]
    w.calls = [kc.KernelCall.MatMul(kc.MatMulCall(kc.rb(0, 0, m * k * 2), kc.rb(1, 0, k * n * 2), kc.rb(2, 0, m * n * 2), m, k, n, BF, 0)),
               kc.KernelCall.AllReduce(kc.AllReduceCall(kc.rb(2, 0, m * n * 2), m * n, BF))]
    img = w.finish()
    x = synth_bf16(m * k, 1.0, 8)
    plain = hb.InferenceSession(backend, img)
    plain.write("x", x)
    plain.execute()
    want = plain.read("y", np.uint16).copy()
    assert want.any()
    addr = hb.InferenceSession(backend, img, addressed=True)
    out, st = addr.execute_addressed([addr.intern_input(x)])
    assert np.array_equal(addr.read("y", np.uint16), want) and st.dispatched == 2
    assert out[0] == hs.label_bytes(want)       # no derivable label: the output is addressed by its bytes
    assert np.array_equal(addr.resolve(out[0], np.uint16), want)
    plain.close()
    addr.close()


def test_add_rms_norm_label_follows_the_reference_operand_list(backend):
    # kernel_call.rs:1612-1616 lists x, gamma, beta for every norm, AddRmsNorm included: by default the label does not
    # see the residual (byte-identical to the reference); HOLO_SESSION_LABEL_RESIDUAL appends it
    b, f = 4, 256
    w = holo.HoloWriter()
    g = synth_bf16(f, 0.1, 3)
    w.add_constant(2, BF, g.tobytes(), by_reference=False)
    nb = b * f * 2
    w.inputs = [holo.Port("x", 0, b * f, BF, [b, f]), holo.Port("r", 1, b * f, BF, [b, f])]
    w.outputs = [holo.Port("y", 3, b * f, BF, [b, f])]
    call = kc.KernelCall.AddRmsNorm(kc.NormCall(kc.rb(0, 0, nb), kc.rb(2, 0, f * 2), kc.NONE, kc.rb(1, 0, nb), kc.rb(3, 0, nb), b, f, 0, 0, 0x3727C5AC, BF))
    w.calls = [call]
    img = w.finish()
    x, r = synth_bf16(b * f, 1.0, 1), synth_bf16(b * f, 1.0, 2)
    op, pr = hs.op_signature(call)
    lx, lr, lg = hs.label_bytes(x), hs.label_bytes(r), hs.label_bytes(g)
    for flag, operands in ((False, [lx, lg]), (True, [lx, lg, lr])):
        sess = hb.InferenceSession(backend, img, addressed=True, label_residual=flag)
        out, _ = sess.execute_addressed([sess.intern_input(x), sess.intern_input(r)])
        assert out[0] == hs.label_derive_boundary(op, pr, operands)
        got, want = sess.read("y", np.uint16), orc.add_rms_norm(x, r, g, b, f, 0x3727C5AC, BF)
        assert norm_max_err(orc.bf16_to_f32(got), orc.bf16_to_f32(want)) <= 1e-2      # parallel sum of squares on the device
        sess.close()


def test_tier_report_under_the_three_policies(backend):
    # crates/hologram-exec/src/coherence.rs:78-225, memory_tier.rs:41-51: bf16 calls are CpuL2, layout-only calls CpuMain,
    # the f32 / i32-indexed ones Device; ForceAllDevice (what this backend executes under) makes every call Device and
    # leaves only the first uploads of inputs and constants as "migrations"; ForceAllCpu has none at all
    cfg = small_cfg(layers=1, batch=2, bucket=128)
    img, _ = dh.build_decoder_step(cfg)
    sess = hb.InferenceSession(backend, img)
    n = sess.n_calls
    dev = sess.tier_report(hs.TIER_FORCE_ALL_DEVICE)
    assert (dev.device_calls, dev.cpu_l1_calls, dev.cpu_l2_calls, dev.cpu_main_calls) == (n, 0, 0, 0)
    assert dev.total_migration_slots > 0
    cpu = sess.tier_report(hs.TIER_FORCE_ALL_CPU)
    assert cpu.cpu_main_calls == n and cpu.total_migration_slots == 0 and cpu.levels_with_migrations == 0
    comp = sess.tier_report(hs.TIER_COMPILED)
    kinds = [sess.call(i).kind for i in range(n)]
    layout = sum(k in (kc.K_GATHER, kc.K_KV_CACHE_WRITE) for k in kinds)
    assert comp.cpu_main_calls == layout and comp.cpu_l2_calls == n - layout and comp.device_calls == 0
    assert comp.total_migration_slots == 0      # nothing is Device-tier in a bf16 graph, so nothing ever leaves the CPU side
    sess.close()


def test_paged_weights_match_the_resident_load(backend):
    # load_paged (session.rs:417): a weightless archive plus a provider; the big constants page in on first use, a
    # budget smaller than the weight set streams them through a bounded window, and the result is bit-identical
    cfg = small_cfg(layers=2, batch=2, bucket=128)
    w_img, info = dh.build_decoder_step(cfg)
    resident = hb.InferenceSession(backend, w_img, addressed=True)
    vals = step_inputs(cfg, info, 50, 50, seed=9)
    labels = [resident.intern_input(vals[p.name]) for p in resident.inputs]
    want_labels, _ = resident.execute_addressed(labels)
    want = resident.read("logits", np.uint16).copy()
    bodies = {holo.fingerprint(bytes(body)): bytes(body) for s_, (dt, body) in info["constants"].items() if len(body) > 256}
    total = sum(len(v) for v in bodies.values())
    store = hb.WeightStore(bodies)
    for budget in (0, total // 3):
        paged = hb.InferenceSession(backend, w_img, weight_store=store, budget=budget)
        outs, st = paged.execute_addressed([paged.intern_input(vals[p.name]) for p in paged.inputs])
        assert np.array_equal(paged.read("logits", np.uint16), want) and outs == want_labels
        assert st.paged_in == len(bodies)
        outs2, st2 = paged.execute_addressed([paged.intern_input(step_inputs(cfg, info, 51, 51, seed=9)[p.name]) for p in paged.inputs])
        # unbounded: every weight paged once and stays; bounded: the window streams them again
        assert (st2.paged_in == len(bodies)) if budget == 0 else (st2.paged_in > len(bodies))
        with pytest.raises(hb.BackendError):
            paged.execute()                       # a paged session executes by labels
        paged.close()
    resident.close()
