"""The cache manager on the host: no page lost, held twice or freed twice, under random orders."""
import random

import numpy as np
import pytest

from return_b200.cache.manager import CacheManager, GroupSpec, KVCapacityError, PagePool
from return_b200.engine.batch import StepEntry, build_host_batch


def test_pool_is_lifo_and_checks_double_free():
    pool = PagePool(4)
    a = pool.take(2)
    assert a == [0, 1] and pool.num_free == 2
    pool.give_back([1])
    assert pool.take(1) == [1]                    # the page freed last comes back first
    with pytest.raises(AssertionError):
        pool.give_back([3])                       # never handed out
    pool.give_back([0])
    with pytest.raises(AssertionError):
        pool.give_back([0])                       # freed twice
    with pytest.raises(KVCapacityError):
        pool.take(9)


def test_append_allocates_by_page_and_all_or_nothing():
    m = CacheManager([GroupSpec("full", 8, 6)], max_requests=3)
    assert m.add("a") == 0 and m.add("b") == 1
    assert m.append("a", 5) == 0 and m.block_table("a", 0) == [0]
    assert m.append("a", 3) == 5 and m.block_table("a", 0) == [0]          # page exactly full
    assert m.append("a", 1) == 8 and m.block_table("a", 0) == [0, 1]
    assert m.pages_needed("b", 33) == [5] and not m.fits("b", 33)
    before = (m.pages_used(), m.length("b"))
    with pytest.raises(KVCapacityError):
        m.append("b", 33)
    assert (m.pages_used(), m.length("b")) == before
    m.append("b", 32)
    assert m.pages_used() == [6]
    m.free("a")
    assert m.pages_used() == [4]
    m.add("c")
    assert m.append("c", 9) == 0 and m.block_table("c", 0) == [1, 0]       # freed pages are used again
    m.check()


def test_slots_run_out_and_come_back():
    m = CacheManager([GroupSpec("full", 4, 4)], max_requests=2)
    m.add(1), m.add(2)
    with pytest.raises(KVCapacityError):
        m.add(3)
    with pytest.raises(KeyError):
        m.add(1)
    s = m.slot(1)
    m.free(1)
    assert m.add(3) == s
    m.check()


def test_window_group_gives_pages_back_while_running():
    full, win = GroupSpec("full", 4, 64), GroupSpec("win", 4, 64, window=6)
    m = CacheManager([full, win], max_requests=2)
    m.add("r")
    m.append("r", 10)                              # nothing cached before: nothing to give back
    assert m.block_table("r", 1) == [0, 1, 2]
    m.append("r", 1)                               # query at 10 sees keys 5..10: block 0 (0..3) is passed
    assert m.block_table("r", 1) == [-1, 1, 2] and m.block_table("r", 0) == [0, 1, 2]
    for _ in range(9):
        m.append("r", 1)
    # length 20: the next query (position 19 was the last appended) ... keys >= 20-1-6+1 = 14 are needed
    assert m.block_table("r", 1)[:3] == [-1, -1, -1] and m.block_table("r", 1)[3] >= 0
    assert m.pages_used()[1] <= 3 and m.pages_used()[0] == 5
    m.check()
    m.free("r")
    assert m.pages_used() == [0, 0]
    m.check()


def test_window_never_frees_a_block_a_query_still_needs():
    P, W = 4, 7
    m = CacheManager([GroupSpec("win", P, 256, window=W)], max_requests=1)
    m.add("r")
    rng = random.Random(0)
    length = 0
    while length < 300:
        n = rng.choice([1, 1, 2, 3, 5, 13])
        start = m.append("r", n)
        assert start == length
        bt = m.block_table("r", 0)
        for q in range(start, start + n):
            for k in range(max(0, q - W + 1), q + 1):
                assert bt[k // P] >= 0, (q, k)
        length += n
        assert m.pages_used()[0] <= (W + 13) // P + 3
        m.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests(seed):
    rng = random.Random(seed)
    groups = [GroupSpec("full", 8, 40), GroupSpec("win", 8, 24, window=rng.choice([5, 16, 33]))]
    m = CacheManager(groups, max_requests=5)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            m.add(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 13, 40])
            if m.fits(rid, n):
                assert m.append(rid, n) == live[rid]
                live[rid] += n
            else:
                used = m.pages_used()
                with pytest.raises(KVCapacityError):
                    m.append(rid, n)
                assert m.pages_used() == used and m.length(rid) == live[rid]
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
            with pytest.raises(KeyError):
                m.free(rid)
        m.check()
        for rid, n in live.items():
            bt = m.block_table(rid, 0)
            assert len(bt) == (n + 7) // 8 and all(p >= 0 for p in bt)
    for rid in list(live):
        m.free(rid)
    assert m.pages_used() == [0, 0] and m.free_slots == 5
    m.check()


def test_host_batch_tables():
    m = CacheManager([GroupSpec("full", 4, 32)], max_requests=4)
    for rid in "abc":
        m.add(rid)
    m.append("a", 6)                                   # earlier step
    entries = []
    for rid, toks, want in (("a", [7], [0]), ("b", [1, 2, 3, 4, 5], [4]), ("c", [9, 8], [0, 1])):
        start = m.append(rid, len(toks))
        entries.append(StepEntry(rid, toks, want, start))
    from return_b200.parts.base import Tiling
    hb = build_host_batch(entries, m, vocab_size=10, tilings={"rows2": Tiling(2), "rows4": Tiling(4, heaviest_first=True)})
    assert hb.num_tokens == 8 and hb.num_segments == 3 and hb.num_want == 4
    assert hb.tokens.tolist() == [7, 1, 2, 3, 4, 5, 9, 8]
    assert hb.pos.tolist() == [6, 0, 1, 2, 3, 4, 0, 1]
    assert hb.tok_seg.tolist() == [0, 1, 1, 1, 1, 1, 2, 2]
    assert hb.cu_q.tolist() == [0, 1, 6, 8] and hb.seg_pos0.tolist() == [6, 0, 0] and hb.seg_kv_len.tolist() == [7, 5, 2]
    assert hb.want_rows.tolist() == [0, 5, 6, 7]
    assert hb.decode_segs.tolist() == [0] and hb.num_multi == 2
    # the tables of row blocks are the ones asked for, by name; no part of the engine knows a kernel's tile
    assert hb.tiles["rows2"].tolist() == [[1, 0], [1, 2], [1, 4], [2, 0]]
    assert hb.tiles["rows4"].tolist() == [[1, 4], [1, 0], [2, 0]]           # most keys before them first
    assert build_host_batch(entries, m, vocab_size=10).tiles == {}
    assert hb.block_tables[0].shape == (3, 2)
    assert hb.block_tables[0][0].tolist() == m.block_table("a", 0)
    assert hb.block_tables[0][2].tolist() == m.block_table("c", 0) + [-1]
    assert hb.seg_slot.tolist() == [m.slot(r) for r in "abc"]
    with pytest.raises(ValueError, match="token ids"):
        build_host_batch(entries, m, vocab_size=9)
    with pytest.raises(ValueError, match="room"):
        build_host_batch([StepEntry("a", [1, 2], [], 3)], m)


def test_fits_all_sums_the_needs_of_a_step():
    """Two requests that each need the last free page: either fits alone, both do not."""
    m = CacheManager([GroupSpec("full", 16, 3)], 4)
    for rid in ("a", "b"):
        m.add(rid)
        m.append(rid, 16)
    assert m.pools[0].num_free == 1
    assert m.fits("a", 1) and m.fits("b", 1)
    assert not m.fits_all(["a", "b"], 1)
    assert m.fits_all(["a"], 1)
    m.append("a", 1)
    with pytest.raises(KVCapacityError):
        m.append("b", 1)
    m.check()


def test_taking_a_slot_calls_the_hooks():
    m = CacheManager([GroupSpec("full", 4, 8)], 2)
    seen = []
    m.on_slot_taken.append(seen.append)
    a = m.add("a")
    b = m.add("b")
    m.free("a")
    c = m.add("c")                       # the slot of "a", taken again: reset again
    assert seen == [a, b, c] and c == a


def test_a_window_group_gets_the_pages_its_requests_can_hold_not_the_whole_pool():
    import torch
    from return_b200.cache.storage import CacheStorage
    from return_b200.parts.base import BuildEnv, KVCacheNeed
    env = BuildEnv(torch.float32, torch.device("cpu"))
    needs = [KVCacheNeed(1, 16, None), KVCacheNeed(1, 16, 24), KVCacheNeed(1, 16, None)]
    st = CacheStorage(needs, 16, 100, 2, env, longest_append=32)
    full, win = st.group_specs
    assert (full.window, full.num_pages) == (None, 100)
    assert (win.window, win.num_pages) == (24, 2 * ((24 + 32 + 15) // 16 + 1))
    assert CacheStorage(needs, 16, 100, 2, env).group_specs[1].num_pages == 100      # longest append unknown
    # two requests that append up to 32 tokens at a time never find the window group short
    m = st.make_manager()
    rng = random.Random(3)
    for rid in ("a", "b"):
        m.add(rid)
    for _ in range(400):
        rid = rng.choice("ab")
        if m.length(rid) > 600:
            m.free(rid)
            m.add(rid)
        n = rng.randint(1, 32)
        if m.pages_needed(rid, n)[0] > m.pools[0].num_free:
            m.free(rid)
            m.add(rid)
        assert m.pages_needed(rid, n)[1] <= m.pools[1].num_free
        m.append(rid, n)
        m.check()
