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
