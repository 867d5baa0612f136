"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice."""
import random

import pytest

from qorvix_b200.cache import CacheManager, FixedStateSpec, OutOfSlots, PageError, PagedKVSpec, native

KV = PagedKVSpec(num_kv_heads=2, head_dim=16)
WIN = PagedKVSpec(num_kv_heads=2, head_dim=16, window=40)
STATE = FixedStateSpec(shape=(4, 8), dtype="float32")


def manager(needs, tokens=256, max_requests=4, allocate=False):
    return CacheManager(needs, max_tokens=tokens, page_size=16, max_requests=max_requests, device="cpu",
                        allocate=allocate)


def test_pool_hands_out_low_ids_first_and_refuses_double_free():
    """The free list of the C++ runtime (csrc/host_runtime.cpp), through its C entry points."""
    L = native.lib()
    pool = L.qvh_pool_create(4)

    def alloc(n):
        out = (native.c_int * max(n, 1))()
        return list(out[:n]) if L.qvh_pool_alloc(pool, n, out) else None

    def free(pages):
        return L.qvh_pool_free(pool, native.ints(pages), len(pages))

    try:
        assert alloc(2) == [0, 1]
        assert alloc(3) is None and L.qvh_pool_num_free(pool) == 2     # all or nothing
        assert free([0]) == 0
        assert alloc(1) == [0]                                          # freed pages are used again at once
        assert free([3]) == -2 or free([3]) < 0                         # never handed out
        assert free([1]) == 0
        assert free([1]) < 0                                            # freed twice
        assert L.qvh_pool_is_held(pool, 0) and not L.qvh_pool_is_held(pool, 1)
    finally:
        L.qvh_pool_destroy(pool)


def test_pages_are_taken_on_page_edges():
    m = manager([(KV, None), (KV, None)])
    m.admit("a")
    assert m.reserve("a", 16) and len(m.block_table("a", 0)) == 1
    m.commit("a", 16)
    assert m.reserve("a", 1) and len(m.block_table("a", 0)) == 2
    m.commit("a", 1)
    assert m.reserve("a", 15) and len(m.block_table("a", 0)) == 2
    m.commit("a", 15)
    assert m.length("a") == 32 and m.free_pages() == 14
    m.check_invariants()
    m.release("a")
    assert m.free_pages() == 16
    m.check_invariants()


def test_groups_by_need_and_shared_cache():
    needs = [(KV, None), (WIN, None), (None, 0), (KV, None), (STATE, None)]
    m = manager(needs, allocate=True)
    assert len(m.groups) == 3 and m.groups[0].layers == [0, 3] and m.groups[1].layers == [1]
    assert m.layer_view(2).group == 0 and m.layer_view(2).tensor.data_ptr() == m.layer_view(0).tensor.data_ptr()
    assert m.layer_view(4).kind == "state" and tuple(m.layer_view(4).tensor.shape) == (5, 4, 8)      # 4 request slots + the scratch slot
    assert tuple(m.layer_view(0).tensor.shape) == (17, 2, 2, 16, 16)       # 16 pages + the scratch page
    with pytest.raises(ValueError):
        manager([(None, 1), (None, None)])


def test_window_pages_go_back_when_the_window_has_passed():
    m = manager([(KV, None), (WIN, None)])
    m.admit("a")
    total = 0
    for n in (30, 30, 30, 1, 1, 40):
        assert m.reserve("a", n)
        m.commit("a", n)
        total += n
        full = m.block_table("a", 0)
        win = m.block_table("a", 1)
        assert all(p >= 0 for p in full) and len(full) == -(-total // 16)
        first_needed = max(0, total - 40 + 1)
        for b, p in enumerate(win):
            assert (p < 0) == ((b + 1) * 16 <= first_needed)
        m.check_invariants()
    assert m.free_pages(1) > m.free_pages(0)
    m.release("a")
    assert m.free_pages(0) == 16 and m.free_pages(1) == 16


def test_reservation_is_all_or_nothing_over_groups():
    m = manager([(KV, None), (WIN, None)], tokens=64)
    m.admit("a"); m.admit("b")
    assert m.reserve("a", 48); m.commit("a", 48)
    before = (m.free_pages(0), m.free_pages(1))
    assert not m.reserve("b", 32)
    assert (m.free_pages(0), m.free_pages(1)) == before and m.block_table("b", 0) == []
    assert m.can_reserve([("b", 16)]) and not m.can_reserve([("b", 16), ("a", 1), (None, 1)])


def test_state_slots_are_zeroed_on_admission_and_reused():
    m = manager([(STATE, None)], max_requests=2, allocate=True)
    s = m.admit("a")
    m.layer_view(0).tensor[s].fill_(7.0)
    m.admit("b")
    with pytest.raises(OutOfSlots):
        m.admit("c")
    m.release("a")
    s2 = m.admit("c")
    assert s2 == s and float(m.layer_view(0).tensor[s2].abs().sum()) == 0.0
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    m = manager([(KV, None), (WIN, None), (KV, None)], tokens=320, max_requests=5)
    live, counter = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.free_slots():
            counter += 1
            rid = f"r{counter}"
            m.admit(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 16, 33])
            before = {g: m.free_pages(g) for g in m.paged_groups()}
            if m.reserve(rid, n):
                m.commit(rid, n)
                live[rid] += n
                assert m.length(rid) == live[rid]
            else:
                assert {g: m.free_pages(g) for g in m.paged_groups()} == before
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
            with pytest.raises(KeyError):
                m.release(rid)
        m.check_invariants()
    for rid in list(live):
        m.release(rid)
    assert all(m.free_pages(g) == m.num_pages for g in m.paged_groups()) and m.free_slots() == 5


@pytest.mark.parametrize("seed", range(3))
def test_decode_rows_kept_between_steps_equal_rows_written_afresh(seed):
    """The rows of a captured decode step are updated in place from step to step; after any order
    of admissions, growth, window release and ends they equal rows written from the block tables."""
    import numpy as np
    rng = random.Random(100 + seed)
    needs = [(KV, None), (WIN, None)]
    m = manager(needs, tokens=640, max_requests=4)
    S, W = 4, 12
    groups = m.paged_groups()
    host = np.full(4 * S + len(groups) * S * W, -7, dtype=np.int32)
    host[4 * S:] = m.scratch_page
    row_epoch = np.zeros(len(groups) * S, dtype=np.int64)
    row_len = np.zeros(len(groups) * S, dtype=np.int32)
    live, counter = [], 0
    for step in range(300):
        op = rng.random()
        if op < 0.15 and m.free_slots():
            counter += 1
            rid = ("req", counter % 3, counter)
            m.admit(rid)
            n = rng.choice([1, 5, 16, 40])
            assert m.reserve(rid, n)
            m.commit(rid, n)
            live.insert(rng.randrange(len(live) + 1), rid)
        elif op < 0.25 and live:
            m.release(live.pop(rng.randrange(len(live))))
        rows = [r for r in live if m.length(r) + 1 <= W * 16 and m.reserve(r, 1)]
        tokens = [rng.randrange(100) for _ in rows]
        m.fill_decode_rows(rows, tokens, S, W, host.ctypes.data, row_epoch.ctypes.data, row_len.ctypes.data)
        want = np.zeros_like(host)
        want[3 * S:4 * S] = m.scratch_slot
        want[4 * S:] = m.scratch_page
        for i, r in enumerate(rows):
            want[i], want[S + i], want[2 * S + i], want[3 * S + i] = tokens[i], m.length(r), m.length(r), m.slot(r)
            for k, g in enumerate(groups):
                t = [p if p >= 0 else m.scratch_page for p in m.block_table(r, g)]
                base = 4 * S + (k * S + i) * W
                want[base:base + len(t)] = t
        assert (host == want).all(), f"step {step}"
        for r in rows:
            m.commit(r, 1)
        for r in [r for r in live if r not in rows]:
            live.remove(r)
            m.release(r)
        m.check_invariants()
