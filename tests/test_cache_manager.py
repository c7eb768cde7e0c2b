"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random orders."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from forge_b200.cache import CacheError, CacheManager, GroupSpec, OutOfPages, PagePool


def test_pool_lifo_reuse_and_double_free():
    pool = PagePool(4)
    a = pool.allocate(3, "x")
    assert a == [0, 1, 2] and pool.num_free == 1
    pool.release(1, "x")
    assert pool.allocate(1, "y") == [1]                   # the page just given back is used again
    with pytest.raises(CacheError, match="held by"):
        pool.release(1, "x")
    pool.release(0, "x")
    with pytest.raises(CacheError, match="freed twice"):
        pool.release(0, "x")
    with pytest.raises(OutOfPages):
        pool.allocate(3, "z")
    pool.check()


def test_append_is_all_or_nothing_across_groups():
    m = CacheManager([GroupSpec("full", 4), GroupSpec("win", 2, window=8)], page_size=4, max_requests=2)
    m.admit("a")
    m.append("a", 8)
    assert m.num_free_pages() == {"full": 2, "win": 0}
    with pytest.raises(OutOfPages):
        m.append("a", 1)                                   # "win" has no page left
    assert m.num_tokens("a") == 8 and m.num_free_pages() == {"full": 2, "win": 0}
    m.check()


def test_slot_mapping_and_block_table():
    m = CacheManager([GroupSpec("g", 8)], page_size=4, max_requests=2)
    m.admit("a"), m.admit("b")
    sa = m.append("a", 3)["g"]
    sb = m.append("b", 5)["g"]
    sa2 = m.append("a", 3)["g"]
    assert sa == [0, 1, 2] and sb == [4, 5, 6, 7, 8] and sa2 == [3, 12, 13]
    assert m.block_table("a", "g") == [0, 3] and m.block_table("b", "g") == [1, 2]
    assert m.slot("a") != m.slot("b")
    m.free("a")
    with pytest.raises(CacheError, match="not admitted"):
        m.free("a")
    m.admit("c")
    assert m.append("c", 1)["g"] == [0]                   # a page that a held, used again
    m.check()


def test_window_gives_pages_back_once_passed():
    m = CacheManager([GroupSpec("full", 16), GroupSpec("win", 16, window=6)], page_size=4, max_requests=1)
    m.admit("a")
    m.append("a", 9)                                       # positions 0..8; next query at 9 reads keys >= 4
    assert m.release_out_of_window("a") == 1
    assert m.block_table("a", "win")[0] == -1 and m.block_table("a", "full")[0] >= 0
    m.append("a", 1)                                       # next query at 10 reads keys >= 5: page 1 still live
    assert m.release_out_of_window("a") == 0
    m.append("a", 3)                                       # next query at 13 reads keys >= 8: page 1 dead
    assert m.release_out_of_window("a") == 1
    assert m.block_table("a", "win")[:2] == [-1, -1]
    m.check()
    m.free("a")
    assert m.num_free_pages() == {"full": 16, "win": 16}


def test_fresh_slots_are_reported_once():
    m = CacheManager([], page_size=4, max_requests=2)
    s = m.admit("a")
    assert m.take_fresh_slots() == [s] and m.take_fresh_slots() == []
    m.free("a")
    assert m.admit("b") == s and m.take_fresh_slots() == [s]
    with pytest.raises(OutOfPages):
        m.admit("c"), m.admit("d")


@settings(max_examples=60, deadline=None)
@given(seed=st.integers(0, 10_000), pages=st.integers(3, 24), page_size=st.sampled_from([1, 4, 16]),
       window=st.sampled_from([None, 5, 33]))
def test_random_orders_keep_every_page_accounted(seed, pages, page_size, window):
    rng = random.Random(seed)
    m = CacheManager([GroupSpec("g", pages, window=window), GroupSpec("h", pages + 2)], page_size, max_requests=4)
    live, next_id = [], 0
    for _ in range(200):
        op = rng.random()
        if op < 0.25 and m.has_free_slot():
            m.admit(next_id)
            live.append(next_id)
            next_id += 1
        elif op < 0.8 and live:
            rid, n = rng.choice(live), rng.randint(1, 3 * page_size)
            before = (m.num_tokens(rid), m.num_free_pages())
            if m.can_append(rid, n):
                slots = m.append(rid, n)
                assert all(len(v) == n and len(set(v)) == n for v in slots.values())
                m.release_out_of_window(rid)
            else:
                with pytest.raises(OutOfPages):
                    m.append(rid, n)
                assert before == (m.num_tokens(rid), m.num_free_pages())
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            m.free(rid)
        m.check()
    for rid in live:
        m.free(rid)
    m.check()
    assert m.num_free_pages() == {"g": pages, "h": pages + 2}


def test_canary_words_around_cache_tensors():
    """Every cache tensor has a guard page in front and behind; a write there (what a kernel following page id -1 or
    num_pages would do) is reported by name.  On the CPU: the storage is plain torch."""
    import torch
    from forge_b200.cache import CacheStorage
    from forge_b200.parts.base import KVCacheSpec, StateSpec
    st = CacheStorage([KVCacheSpec(2, 8), StateSpec((5,))], [None, None], page_size=4, pages_per_group=3, max_requests=2,
                      dtype=torch.float32, device=torch.device("cpu"))
    assert st.layers[0].kv.shape == (3, 2, 2, 4, 8) and st.layers[0].kv.is_contiguous() and not st.layers[0].kv.any()
    assert st.check_canaries() == []
    st.layers[0].kv[2, 1, 1, 3, 7] = 1.0                       # the last element inside: fine
    assert st.check_canaries() == []
    whole = st._guarded[0][1]
    whole[4, 0, 0, 0, 0] = 3.0                                  # "page 3" of 3: the guard behind
    assert st.check_canaries() == ["keys/values of run 0 (the guard behind it)"]
    whole[4].view(torch.uint8).fill_(st.CANARY_BYTE)
    st._guarded[1][1][0, 2] = 1.0                               # "slot -1" of the state rows
    assert st.check_canaries() == ["state of run 1 (the guard before it)"]
