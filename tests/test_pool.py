"""The label-keyed buffer pool's residency rules on host memory (no GPU): the same table logic that
runs over cudaMalloc'd buffers, through the C ABI. Follows crates/hologram-exec/src/buffer.rs
(rebind_reset :352, acquire_buf :528, store_unbound :683, retain :710, steal_transient :731,
lease / release :795-836, bindable_input :858, page_and_bind_group :650) and the witnesses of
crates/hologram-exec/tests/lease.rs."""
import blake3
import numpy as np
import pytest

import hologram_b200 as hb
from hologram_b200 import session as hs


def lab(data):
    return hs.label_bytes(np.ascontiguousarray(data))


@pytest.fixture
def pool():
    p = hb.DevicePool(None)
    yield p
    p.close()


def test_store_resolve_and_two_generation_rotation(pool):
    a, b = np.arange(1000, dtype=np.uint8), np.arange(1000, dtype=np.uint8)[::-1].copy()
    la, lb = lab(a), lab(b)
    pool.store_unbound(la, a)
    assert pool.resident(la) and pool.bindable_input(la) and not pool.resident(lb)
    assert np.array_equal(pool.resolve(la), a) and pool.resolve(lb) is None
    pool.rebind_reset(4)                       # walk 1: `a` ages into the previous generation
    assert pool.resident(la) and not pool.bindable_input(la)
    assert pool.bind_resident(0, la) and pool.slot(0)[1] == 1000
    pool.store_unbound(la, a)                  # re-interning promotes it: bindable again, no second buffer
    assert pool.bindable_input(la) and pool.stats().owned_bytes == 1024
    pool.rebind_reset(4)
    pool.rebind_reset(4)                       # two rotations without a touch: gone, its buffer released
    assert not pool.resident(la) and pool.resolve(la) is None
    assert pool.stats().released == 1


def test_released_buffers_are_reused_best_fit_and_zeroed(pool):
    pool.rebind_reset(4)
    pool.bind_fresh(0, 4096)
    pool.bind_fresh(1, 100)
    pool.write_slot(0, np.full(4096, 0xAB, dtype=np.uint8))
    p0 = pool.slot(0)[0]
    pool.rebind_reset(4)                       # both were slot-only scratch: released
    assert pool.stats().released == 2
    pool.bind_fresh(2, 3000)                   # 3008 <= 4096 <= 2 x 3008: reuses the large buffer...
    assert pool.slot(2)[0] == p0 and pool.stats().owned_bytes == 4096 + 128
    pool.retain(2, lab(b"x"))
    assert not np.any(pool.resolve(lab(b"x")))  # ... zero-filled, the old bytes do not show
    pool.bind_fresh(3, 1000)                   # 1024 bytes: the 128-byte one is too small, the other is taken: new
    assert pool.stats().owned_bytes == 4096 + 128 + 1024


def test_lease_is_ownership_not_recency(pool):
    v = np.arange(256, dtype=np.uint8)
    l, ghost = lab(v), lab(b"never stored")
    pool.store_unbound(l, v)
    assert not pool.lease(ghost) and pool.lease(l) and pool.lease(l)      # refcounted
    for _ in range(5):
        pool.rebind_reset(2)
    assert np.array_equal(pool.resolve(l), v) and pool.bindable_input(l) and pool.stats().leased == 1
    assert pool.release(l) and pool.resident(l) and pool.stats().leased == 1
    assert pool.release(l) and not pool.release(l) and pool.stats().leased == 0
    assert pool.bindable_input(l)              # demoted into the current generation: consumable once more
    pool.rebind_reset(2)
    pool.rebind_reset(2)
    assert not pool.resident(l)


def test_steal_needs_unique_ownership(pool):
    v = np.arange(512, dtype=np.uint8)
    l = lab(v)
    pool.rebind_reset(4)
    pool.store_unbound(l, v)
    assert pool.bind_resident(0, l)
    assert pool.bind_resident(3, l)            # a second reader outside the allowed set
    assert not pool.steal_transient(l, [0, 1], 1)
    pool.rebind_reset(4)
    pool.store_unbound(l, v)
    pool.bind_resident(0, l)
    assert pool.lease(l) and not pool.steal_transient(l, [0, 1], 1)      # a lease is a borrow: no move
    assert pool.release(l)
    pool.bind_fresh(2, 512)
    pool.retain(2, lab(b"alias"))
    assert pool.steal_transient(l, [0, 1], 1)                             # sole owner now: moved
    assert not pool.resident(l) and pool.slot(1)[0] == pool.slot(0)[0]
    pinned = lab(b"const")
    pool.pin_bytes(pinned, np.frombuffer(b"const", dtype=np.uint8))
    assert not pool.steal_transient(pinned, [0], 1) and pool.lease(pinned) and not pool.release(pinned)


def test_paged_weights_stay_within_the_budget(pool):
    bodies = {i: np.full(1000, i, dtype=np.uint8) for i in range(4)}
    fps = {i: blake3.blake3(b.tobytes()).digest() for i, b in bodies.items()}
    labels = {i: b"blake3:" + fps[i].hex().encode() for i in bodies}
    store = hb.WeightStore({fps[i]: bodies[i].tobytes() for i in bodies})
    for i in bodies:
        pool.pin_lazy(labels[i], fps[i], 1000)
    pool.set_lazy_budget(2000)
    assert not pool.resident(labels[0]) and not pool.lease(labels[0])     # the pager owns a lazy weight's lifecycle
    pool.rebind_reset(4)
    assert pool.page_and_bind([(0, labels[0])], store) and pool.page_and_bind([(1, labels[1])], store)
    assert pool.stats().lazy_resident_bytes == 2000 and pool.stats().pages_in == 2
    assert np.array_equal(pool.resolve(labels[0]), bodies[0])
    pool.rebind_reset(4)                                                  # paged weights survive the rotation
    assert pool.page_and_bind([(0, labels[0])], store) and pool.stats().pages_in == 2     # a hit pages nothing
    assert pool.page_and_bind([(2, labels[2])], store)                    # evicts the least recently used: weight 1
    assert pool.resident(labels[0]) and not pool.resident(labels[1]) and pool.stats().lazy_resident_bytes == 2000
    # a group is resident together even when it exceeds the budget; nothing of the group is evicted for the group
    assert pool.page_and_bind([(0, labels[1]), (1, labels[2]), (2, labels[3])], store)
    assert all(pool.resident(labels[i]) for i in (1, 2, 3)) and pool.stats().lazy_resident_bytes == 3000
    # the provider cannot serve it: fail closed, the weight stays non-resident
    missing = b"blake3:" + bytes(32).hex().encode()
    pool.pin_lazy(missing, bytes(32), 64)
    assert not pool.page_and_bind([(3, missing)], store) and not pool.resident(missing)
