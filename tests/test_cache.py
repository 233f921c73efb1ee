"""Bookkeeping of the cache on the CPU: no slot or block is lost, held twice or freed twice."""
import random

import pytest
import torch

from vlrf_b200.cache import BLOCK_TOKENS, CacheError, FreeList, KVNeed, SequenceCache, StateNeed


def make(max_tokens=512, max_seq_len=256, n_slots=None, needs=None):
    needs = needs if needs is not None else [KVNeed(2, 16)] * 3
    return SequenceCache(needs, max_tokens=max_tokens, max_seq_len=max_seq_len, dtype=torch.float32, device="cpu",
                         n_slots=n_slots)


def test_free_list_refuses_misuse():
    f = FreeList(4, "thing")
    a = f.take(3)
    assert sorted(a) == [0, 1, 2] and f.n_free == 1
    with pytest.raises(CacheError, match="out of things"):
        f.take(2)
    f.give([a[0]])
    with pytest.raises(CacheError, match="not held"):
        f.give([a[0]])                     # freed twice
    with pytest.raises(CacheError, match="not held"):
        f.give([3])                        # never taken
    with pytest.raises(CacheError, match="does not exist"):
        f.give([9])
    with pytest.raises(CacheError, match="not held"):
        f.give([a[1], a[1]])               # twice in one call
    f.check()


def test_freed_ids_are_used_again_first():
    f = FreeList(8)
    a = f.take(5)
    f.give([a[2]])
    assert f.take(1) == [a[2]]


def test_max_tokens_sizes_the_pool_in_blocks_of_64():
    c = make(max_tokens=130)
    assert BLOCK_TOKENS == 64 and c.n_blocks == 3 and c.max_tokens == 192 and c.n_slots == 3
    v = c.view(0)
    assert v.k.shape == (3, 2, 64, 16) and v.v.shape == v.k.shape and v.block_table.shape == (3, 4)


def test_growth_takes_blocks_and_release_returns_all():
    c = make(max_tokens=512)
    s = c.acquire()
    c.reserve(s, 5); c.advance(s, 5)
    assert len(c._groups[0].blocks_of(s)) == 1
    c.reserve(s, 64); c.advance(s, 59)
    assert len(c._groups[0].blocks_of(s)) == 1
    c.reserve(s, 65); c.advance(s, 1)
    assert len(c._groups[0].blocks_of(s)) == 2 and c.lengths[s] == 65
    c.check()
    c.release(s)
    assert c._groups[0].pool.n_free == c.n_blocks and c.slots.n_free == c.n_slots
    c.check()
    with pytest.raises(CacheError, match="not held"):
        c.release(s)


def test_cache_full_is_an_error_and_changes_nothing():
    c = make(max_tokens=128, max_seq_len=256)
    a, b = c.acquire(), c.acquire()
    c.reserve(a, 64); c.advance(a, 64)
    c.reserve(b, 10); c.advance(b, 10)
    before = c._groups[0].table_host.copy()
    with pytest.raises(CacheError, match="cache full"):
        c.reserve(a, 65)
    assert (c._groups[0].table_host == before).all()
    c.check()
    with pytest.raises(CacheError, match="exceeds"):
        c.reserve(b, 257)
    with pytest.raises(CacheError, match="out of cache slots"):
        c.acquire()


def test_groups_have_storage_of_their_own():
    needs = [KVNeed(2, 16), KVNeed(2, 16, "window", 70), KVNeed(2, 16), StateNeed((4, 3)), None, KVNeed(1, 32)]
    c = make(max_tokens=1024, max_seq_len=512, needs=needs)
    assert len(c._groups) == 4
    assert c.view(0).k.data_ptr() != c.view(2).k.data_ptr()          # two layers of one group
    assert c.view(0).block_table.data_ptr() == c.view(2).block_table.data_ptr()
    assert c.view(1).block_table.data_ptr() != c.view(0).block_table.data_ptr()
    assert c.view(3).state.shape == (c.n_slots, 4, 3) and c.view(5).k.shape[1:] == (1, 64, 32)
    with pytest.raises(CacheError, match="keeps nothing"):
        c.view(4)
    s = c.acquire()
    c.reserve(s, 200); c.advance(s, 200)
    full, win = c._groups[0], c._groups[1]
    assert len(full.blocks_of(s)) == 4
    # the next query (position 200) sees keys 131…200: block 0 and 1 (positions < 128) are gone
    assert [i for i in range(8) if win.table_host[s, i] >= 0] == [2, 3]
    c.check()
    c.release(s)
    c.check()


def test_state_is_zeroed_when_a_slot_is_taken():
    c = make(needs=[StateNeed((5,))])
    s = c.acquire()
    c.view(0).state[s] = 7.0
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and float(c.view(0).state[s2].abs().sum()) == 0.0


def test_random_walk_keeps_the_invariants():
    rng = random.Random(3)
    c = make(max_tokens=64 * 20, max_seq_len=300)
    live = {}
    for _ in range(2000):
        r = rng.random()
        if r < 0.25 and c.slots.n_free:
            try:
                s = c.acquire()
                n = rng.randint(1, 150)
                c.reserve(s, n); c.advance(s, n)
                live[s] = n
            except CacheError:
                c.release(s)
        elif r < 0.8 and live:
            s = rng.choice(list(live))
            if live[s] < 300:
                try:
                    c.reserve(s, live[s] + 1); c.advance(s, 1)
                    live[s] += 1
                except CacheError:
                    pass
        elif live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        c.check()
        held = sum((n + 63) // 64 for n in live.values())
        assert c._groups[0].pool.n_held == held
    for s in list(live):
        c.release(s)
    c.check()
    assert c._groups[0].pool.n_free == c.n_blocks
