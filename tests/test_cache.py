"""The cache manager (CPU): pages, tables, groups, window release, slots."""
import random

import pytest
import torch

from zllm_b200.cache import CacheManager, NO_PAGE
from zllm_b200.errors import MemoryError_
from zllm_b200.parts import KVCacheSpec, StateSpec


def make(n_pages=16, bs=4, slots=4, max_len=64, needs=None, allocate=False):
    needs = needs or [(KVCacheSpec(2, 16), None), (KVCacheSpec(2, 16), None)]
    return CacheManager(needs, bs, n_pages, slots, max_len, torch.float32, "cpu", allocate=allocate)


def test_layers_with_equal_needs_share_a_group():
    cm = make(needs=[(KVCacheSpec(2, 16), None), (KVCacheSpec(2, 16, window=8), None), (KVCacheSpec(2, 16), None),
                     (KVCacheSpec(2, 16), 0), (None, None), (StateSpec((3, 5)), None)], allocate=True)
    assert len(cm.groups) == 2
    assert cm.groups[0].entries == [0, 2] and cm.groups[1].entries == [1]
    assert cm.view(0).k_pages.shape == (16, 2, 4, 16) and cm.view(2).group == 0 and cm.view(1).window == 8
    assert cm.view(3) is None and cm.view(4) is None           # reads entry 0's cache / needs none
    assert cm.view(5).state.shape == (4, 3, 5)
    assert cm.view(0).k_pages.data_ptr() != cm.view(2).k_pages.data_ptr()


def test_slot_zero_and_page_zero_first_and_tables_grow():
    cm = make()
    s = cm.admit()
    assert s == 0 and cm.admit() == 1
    assert cm.pages_short(s, 9) == [3]
    assert cm.ensure(s, 9)
    assert list(cm.groups[0].table[s, :4]) == [0, 1, 2, NO_PAGE]
    cm.advance(s, 9)
    assert cm.pages_short(s, 12) == [0] and cm.pages_short(s, 13) == [1]
    assert cm.free_pages() == [13]
    cm.check_integrity()


def test_all_or_nothing_and_exhaustion():
    cm = make(n_pages=4)
    a, b = cm.admit(), cm.admit()
    assert cm.ensure(a, 12)            # 3 pages
    assert not cm.can_fit([(b, 8)])
    assert not cm.ensure(b, 8)         # needs 2, 1 free: nothing is taken
    assert cm.free_pages() == [1]
    assert cm.ensure(b, 4)
    assert cm.free_pages() == [0]
    cm.check_integrity()
    cm.free_slot(a)
    assert cm.free_pages() == [3] and cm.ensure(b, 16)
    cm.check_integrity()


def test_double_free_and_dead_slot_are_errors():
    cm = make()
    s = cm.admit()
    cm.ensure(s, 5)
    cm.free_slot(s)
    with pytest.raises(MemoryError_, match="freed twice"):
        cm.free_slot(s)
    with pytest.raises(MemoryError_, match="not live"):
        cm.ensure(s, 3)
    with pytest.raises(MemoryError_, match="exceed"):
        cm.ensure(cm.admit(), 65)


def test_pages_are_used_again():
    cm = make(n_pages=3)
    a = cm.admit()
    cm.ensure(a, 12)
    held = set(int(p) for p in cm.groups[0].table[a, :3])
    cm.free_slot(a)
    b = cm.admit()
    cm.ensure(b, 12)
    assert set(int(p) for p in cm.groups[0].table[b, :3]) == held
    cm.check_integrity()


def test_window_group_gives_pages_back_during_the_request():
    cm = make(n_pages=8, bs=4, max_len=64, needs=[(KVCacheSpec(1, 16, window=6), None), (KVCacheSpec(1, 16), None)])
    s = cm.admit()
    win, full = cm.groups
    pos = 0
    for n in (5, 1, 1, 7, 2, 1, 1, 1, 9):
        assert cm.ensure(s, pos + n)
        pos += n
        cm.advance(s, pos)
        cm.check_integrity()
        # the next query (at pos) sees keys pos-5..pos: every page holding one of them is there
        for key in range(max(0, pos - 6 + 1), pos):
            assert win.table[s, key // 4] != NO_PAGE
        # and nothing older is kept
        first_needed = max(0, pos - 6 + 1) // 4
        assert all(win.table[s, b] == NO_PAGE for b in range(first_needed))
        assert all(full.table[s, b] != NO_PAGE for b in range(-(-pos // 4)))
    assert win.pool.n_free() >= 8 - 3 and full.pool.n_free() == 8 - 7
    cm.free_slot(s)
    assert cm.free_pages() == [8, 8]
    cm.check_integrity()


def test_state_slots_start_at_zero():
    cm = make(needs=[(StateSpec((2, 3)), None)], allocate=True)
    s = cm.admit()
    cm.view(0).state[s] += 5.0
    cm.free_slot(s)
    s2 = cm.admit()
    assert s2 == s and float(cm.view(0).state[s2].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_double_a_page(seed):
    rng = random.Random(seed)
    cm = make(n_pages=24, bs=4, slots=5, max_len=48,
              needs=[(KVCacheSpec(1, 16), None), (KVCacheSpec(1, 16, window=10), None)])
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and cm.has_free_slot():
            s = cm.admit()
            assert s not in live
            live[s] = 0
        elif op < 0.85 and live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 13])
            new_len = min(48, live[s] + n)
            if new_len > live[s]:
                before = cm.free_pages()
                if cm.ensure(s, new_len):
                    live[s] = new_len
                    cm.advance(s, new_len)
                else:
                    assert cm.free_pages() == before          # a refused growth takes nothing
        elif op < 0.92 and live:
            s = rng.choice(list(live))
            n = rng.randint(0, live[s])
            before = cm.free_pages()
            try:
                cm.truncate(s, n)
                live[s] = n
            except MemoryError_:
                assert cm.free_pages() == before              # a refused truncation changes nothing
        elif live:
            s = rng.choice(list(live))
            cm.free_slot(s)
            del live[s]
        cm.check_integrity()
        for s, n in live.items():
            assert cm.length[s] == n
    for s in list(live):
        cm.free_slot(s)
    cm.check_integrity()
    assert cm.free_pages() == [24, 24] and len(cm.free_slots) == 5


def test_truncate_gives_back_the_pages_beyond_and_growth_continues_there():
    cm = make(n_pages=12, bs=4, max_len=48, needs=[(KVCacheSpec(1, 16), None)])
    s = cm.admit()
    assert cm.ensure(s, 21)
    cm.advance(s, 21)
    assert cm.free_pages() == [12 - 6]
    cm.truncate(s, 9)                                # positions 0..8 stay: 3 pages
    cm.check_integrity()
    assert cm.length[s] == 9 and cm.free_pages() == [12 - 3]
    assert all(cm.groups[0].table[s, b] != NO_PAGE for b in range(3)) and cm.groups[0].table[s, 3] == NO_PAGE
    assert cm.ensure(s, 14)
    cm.advance(s, 14)
    cm.check_integrity()
    assert cm.free_pages() == [12 - 4]
    cm.truncate(s, 14)                               # nothing to do
    with pytest.raises(MemoryError_):
        cm.truncate(s, 15)
    cm.truncate(s, 0)
    cm.check_integrity()
    assert cm.free_pages() == [12] and cm.length[s] == 0
    cm.free_slot(s)
    with pytest.raises(MemoryError_):
        cm.truncate(s, 0)


def test_truncate_with_a_window_and_with_state():
    cm = make(n_pages=8, bs=4, max_len=64, needs=[(KVCacheSpec(1, 16, window=6), None), (KVCacheSpec(1, 16), None)])
    s = cm.admit()
    assert cm.ensure(s, 30)
    cm.advance(s, 30)                                # the window group holds the pages of keys 25..29 only
    cm.check_integrity()
    cm.truncate(s, 29)                               # the query at 29 sees keys 24..28: page 6 is still there
    cm.check_integrity()
    with pytest.raises(MemoryError_, match="given back"):
        cm.truncate(s, 20)                           # keys 15..19 went back to the pool long ago
    assert cm.length[s] == 29
    cm.truncate(s, 0)                                # a reset is always possible
    cm.check_integrity()
    assert cm.free_pages() == [8, 8]
    assert cm.ensure(s, 5)
    cm.advance(s, 5)
    cm.check_integrity()
    st = make(needs=[(StateSpec((3,)), None), (KVCacheSpec(1, 16), None)], allocate=True)
    s2 = st.admit()
    assert st.ensure(s2, 6)
    st.advance(s2, 6)
    st.view(0).state[s2] += 1.0
    with pytest.raises(MemoryError_, match="state"):
        st.truncate(s2, 3)
    st.truncate(s2, 0)
    assert float(st.view(0).state[s2].abs().sum()) == 0.0


def shared(n_pages=12, bs=4, slots=4, max_len=64):
    return CacheManager([(KVCacheSpec(1, 16), None), (KVCacheSpec(2, 16), None)], bs, n_pages, slots, max_len,
                        torch.float32, "cpu", allocate=False, prefix_sharing=True)


def fill(cm, slot, tokens, upto=None):
    upto = len(tokens) if upto is None else upto
    assert cm.ensure(slot, upto)
    cm.advance(slot, upto)
    cm.register_prefix(slot, tokens, upto)


def test_a_second_request_takes_over_the_full_pages_of_a_prefix():
    cm = shared()
    a = list(range(100, 119))                        # 19 tokens: 4 full pages of 4 and 3 more
    s0 = cm.admit()
    assert cm.adopt_prefix(s0, a) == 0               # nothing registered yet
    fill(cm, s0, a)
    cm.check_integrity()
    s1 = cm.admit()
    b = a[:13] + [7, 8, 9]                           # the same first 3 pages, then other tokens
    assert cm.adopt_prefix(s1, b) == 12 and cm.length[s1] == 12
    for g in cm.groups:
        assert list(g.table[s1, :3]) == list(g.table[s0, :3]) and g.table[s1, 3] == NO_PAGE
    cm.check_integrity()
    assert cm.free_pages() == [12 - 5, 12 - 5]       # s1 holds no page of its own yet
    fill(cm, s1, b)
    cm.check_integrity()
    assert cm.free_pages() == [12 - 6, 12 - 6]
    # the block with the LAST token is never taken over: one position is left to compute
    s2 = cm.admit()
    assert cm.adopt_prefix(s2, a[:16]) == 12
    assert cm.adopt_prefix(s2, a[:16]) == 0          # only into an empty slot
    cm.free_slot(s2)
    cm.free_slot(s0)                                 # shared pages stay with s1; a's 4th page stays findable
    cm.check_integrity()
    assert cm.free_pages() == [12 - 4, 12 - 4]       # s1: 3 shared + 1 own full... and its partial page
    cm.free_slot(s1)
    cm.check_integrity()
    assert cm.free_pages() == [12, 12]               # everything is free or reclaimable
    s3 = cm.admit()
    assert cm.adopt_prefix(s3, a) == 16              # and still findable after everybody left
    assert cm.prefix_hits == 12 + 12 + 16
    cm.check_integrity()


def test_registered_pages_are_reclaimed_oldest_first_when_the_stack_is_empty():
    cm = shared(n_pages=6, bs=4)
    a, b = list(range(10, 19)), list(range(50, 59))  # 2 full pages + 1 token each
    for toks in (a, b):
        s = cm.admit()
        fill(cm, s, toks)
        cm.free_slot(s)
    cm.check_integrity()
    assert cm.free_pages() == [6, 6] and len(cm.groups[0].pool.free) == 2   # 4 registered pages wait to be found
    s = cm.admit()
    assert cm.ensure(s, 13)                          # 4 pages: the 2 free ones and a's two (the oldest)
    cm.advance(s, 13)
    cm.check_integrity()
    t = cm.admit()
    assert cm.adopt_prefix(t, a) == 0                # a's pages are gone
    assert cm.adopt_prefix(t, b) == 8                # b's are still there
    cm.check_integrity()
    assert not cm.ensure(t, 20)                      # 3 more pages, none left
    cm.free_slot(s)
    assert cm.ensure(t, 20)
    cm.check_integrity()


def test_truncate_into_a_shared_page_is_refused_and_a_sole_holder_unregisters():
    cm = shared()
    a = list(range(30, 47))
    s0 = cm.admit()
    fill(cm, s0, a)
    s1 = cm.admit()
    assert cm.adopt_prefix(s1, a) == 16
    with pytest.raises(MemoryError_, match="shared"):
        cm.truncate(s1, 6)
    cm.truncate(s1, 8)                               # at a page's edge: fine
    cm.check_integrity()
    cm.free_slot(s0)
    cm.truncate(s1, 6)                               # now the only holder: the page stops being findable
    cm.check_integrity()
    s2 = cm.admit()
    assert cm.adopt_prefix(s2, a) == 4
    cm.check_integrity()


@pytest.mark.parametrize("seed", range(4))
def test_random_orders_with_shared_prefixes(seed):
    rng = random.Random(100 + seed)
    cm = shared(n_pages=20, bs=4, slots=5, max_len=40)
    stems = [[rng.randrange(50) for _ in range(40)] for _ in range(3)]
    live = {}
    for _ in range(500):
        op = rng.random()
        if op < 0.3 and cm.has_free_slot():
            s = cm.admit()
            stem = rng.choice(stems)
            cut = rng.randrange(1, 40)
            toks = stem[:cut] + [rng.randrange(50) for _ in range(rng.randrange(1, 40 - cut + 1))]
            n = cm.adopt_prefix(s, toks)
            assert n % 4 == 0 and n < len(toks) and cm.length[s] == n
            live[s] = toks
        elif op < 0.85 and live:
            s = rng.choice(list(live))
            new_len = min(len(live[s]), cm.length[s] + rng.choice([1, 1, 2, 5, 13]))
            if new_len > cm.length[s] and cm.ensure(s, new_len):
                cm.advance(s, new_len)
                cm.register_prefix(s, live[s], new_len)
        elif op < 0.9 and live:
            s = rng.choice(list(live))
            try:
                cm.truncate(s, rng.randint(0, cm.length[s]))
            except MemoryError_:
                pass
        elif live:
            s = rng.choice(list(live))
            cm.free_slot(s)
            del live[s]
        cm.check_integrity()
        # a shared page holds the same tokens for all its holders
        for g in cm.groups:
            for p in range(g.pool.num_pages):
                hs = sorted(g.pool.holders[p])
                if len(hs) > 1:
                    blocks = [list(g.table[s]).index(p) for s in hs]
                    assert len(set(blocks)) == 1
                    b = blocks[0]
                    assert len({tuple(live[s][:4 * b + 4]) for s in hs}) == 1
    for s in list(live):
        cm.free_slot(s)
    cm.check_integrity()
    assert cm.free_pages() == [20, 20]


def test_a_hash_collision_is_not_a_match():
    from zllm_b200.cache.manager import PagePool
    pool = PagePool(4)
    p = pool.alloc(0)
    pool.register(p, 1234, (0, (1, 2, 3, 4)))
    assert pool.lookup(1234, (0, (1, 2, 3, 4))) == p
    assert pool.lookup(1234, (0, (9, 2, 3, 4))) is None      # the same hash, other tokens
    q = pool.alloc(1)
    pool.register(q, 1234, (0, (9, 2, 3, 4)))                # the hash is taken: q stays unregistered
    assert pool.hash_of[q] is None and pool.lookup(1234, (0, (1, 2, 3, 4))) == p
