"""Host-side bookkeeping of the cache: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from inference_engine_rust_b200.cache import (Cache, CacheError, CacheFull, IndexPool, KVRequest,
                                              StateRequest)


def make(max_tokens=64 * 8, max_seq_len=512, max_sequences=4, window=None, extra=None):
    reqs = {0: KVRequest(2, 16, None), 1: KVRequest(2, 16, None), 2: KVRequest(2, 16, window or 100)}
    if extra:
        reqs.update(extra)
    return Cache(reqs, max_tokens=max_tokens, max_seq_len=max_seq_len, max_sequences=max_sequences,
                 dtype=torch.float32, device="cpu")


def test_index_pool():
    p = IndexPool(3, "slot")
    a, b, c = p.alloc(), p.alloc(), p.alloc()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheFull):
        p.alloc()
    p.free(b)
    with pytest.raises(CacheError):
        p.free(b)                       # freed twice
    with pytest.raises(CacheError):
        p.free(7)                       # never handed out
    assert p.alloc() == b               # the one just returned is used again first
    p.check()
    with pytest.raises(CacheFull):
        p.alloc_many(2)


def test_groups_by_need():
    c = make()
    assert len(c.kv_groups) == 2
    full = [g for g in c.kv_groups if g.req.window is None][0]
    ring = [g for g in c.kv_groups if g.req.window is not None][0]
    assert full.layers == (0, 1) and ring.layers == (2,)
    assert full.k.shape == (2, 8, 2, 64, 16) and ring.k.shape == (1, 8, 2, 64, 16)
    assert full.ring_pages == full.table_width == 8 and ring.ring_pages == 2      # ceil(100 / 64)
    assert c.layer_view(2).group is ring and c.layer_view(0).index == 0 and c.layer_view(1).index == 1


def test_pages_follow_lengths_and_come_back():
    c = make()
    full = [g for g in c.kv_groups if g.req.window is None][0]
    ring = [g for g in c.kv_groups if g.req.window is not None][0]
    s0, s1 = c.open_sequence(), c.open_sequence()
    c.reserve(s0, 65)
    c.reserve(s1, 300)
    assert len(full.pages_of(s0)) == 2 and len(full.pages_of(s1)) == 5
    assert len(ring.pages_of(s0)) == 2 and len(ring.pages_of(s1)) == 2           # the ring stops growing
    assert full.pages.free_count == 1
    assert list(full.table_host[s0, :3]) == full.pages_of(s0) + [-1]
    c.advance(s0, 65); c.advance(s1, 300)
    assert c.tokens_held() == 128 + 320
    c.check()
    with pytest.raises(CacheFull):
        c.reserve(s0, 65 + 128)         # needs 2 more pages, one is free
    c.check()
    c.close_sequence(s1)
    assert full.pages.free_count == 6 and (full.table_host[s1] == -1).all()
    c.reserve(s0, 300)
    c.check()
    with pytest.raises(CacheError):
        c.close_sequence(s1)            # closed twice
    with pytest.raises(CacheError):
        c.reserve(s1, 10)
    with pytest.raises(CacheError):
        c.length(s1)
    c.close_sequence(s0)
    assert full.pages.free_count == 8 and ring.pages.free_count == 8 and c.slots.free_count == 4
    c.check()


def test_longest_sequence_and_slots():
    c = make(max_tokens=64 * 8, max_seq_len=200, max_sequences=2)
    s = c.open_sequence()
    with pytest.raises(CacheFull):
        c.reserve(s, 201)
    c.reserve(s, 200)
    c.open_sequence()
    with pytest.raises(CacheFull):
        c.open_sequence()
    c.check()


def test_slot_reuse_resets_length_and_state():
    c = make(extra={5: StateRequest((3,), torch.float32)})
    st = c.layer_view(5)
    s = c.open_sequence()
    c.reserve(s, 10); c.advance(s, 10)
    st.state[s] += 7.0
    assert c.length(s) == 10
    c.close_sequence(s)
    s2 = c.open_sequence()
    assert s2 == s and c.length(s2) == 0 and float(st.state[s2].abs().sum()) == 0.0


def test_random_open_close_never_loses_anything():
    rnd = random.Random(0)
    c = make(max_tokens=64 * 40, max_seq_len=640, max_sequences=9)
    live = {}
    for _ in range(600):
        op = rnd.random()
        if op < 0.35 and c.slots.free_count:
            live[c.open_sequence()] = 0
        elif op < 0.8 and live:
            s = rnd.choice(list(live))
            n = live[s] + rnd.randint(1, 90)
            try:
                c.reserve(s, n)
                c.advance(s, n - live[s])
                live[s] = n
            except CacheFull:
                pass
        elif live:
            s = rnd.choice(list(live))
            c.close_sequence(s)
            del live[s]
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
            for g in c.kv_groups:
                assert len(g.pages_of(s)) == g.pages_needed(n)
    for s in list(live):
        c.close_sequence(s)
    c.check()
    assert all(g.pages.free_count == g.n_pages for g in c.kv_groups)
