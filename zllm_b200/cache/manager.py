"""The cache manager: pages of keys and values with a block table per request,
groups of layers with pools of their own, and slots for per-request state of
fixed size.

Behaviour after the reference's ``BlockState`` / ``BatchedDecoder`` paging (zllm
src/backend/gpu/mod.rs:1876-2055): a page holds ``block_size`` positions
(default 16, mod.rs:1839-1841); a page id addresses the same page in every
layer of its group (mod.rs:1973-1978); the free list is a stack that hands out
page 0 first (mod.rs:1985); ``ensure`` grows a request's table page by page
(mod.rs:2013-2024); ``free_slot`` gives every page back (mod.rs:2030-2040);
``free_pages``/``can_fit``/``pages_short`` answer the scheduler (mod.rs:2043-2055);
request slots are a stack, slot 0 first, kept for the request's life
(src/backend/gpu/batch.rs:65-66).

Beyond the reference (whose layers all have identical pools): layers are put
into *groups* by what they need -- (kv heads, head size, window) -- and each
group has its own pool and tables under the shared slot id.  A group with a
window gives pages back during the request, as soon as every position of the
page has fallen out of the window of the next query.  Per-request state of
fixed size lives in arrays [slots, ...] indexed by the slot id, zeroed at
admission.

Within a page the layout is [kv head][position][head_dim], so the keys of one
head in one page are one contiguous run.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import ConfigError, MemoryError_
from ..parts.base import KVCacheSpec, StateSpec

NO_PAGE = -1


class PagePool:
    """Free stack of page ids; every page knows who holds it (integrity checks are cheap).

    A page is held by one request, or -- when it is registered under the hash of the token
    prefix it completes (``register``) -- by any number of requests that share that prefix.  A
    registered page whose last holder let go keeps its contents and stays findable until the
    free stack is empty and it is the least recently released one (mod.rs:1912-1929).
    """

    def __init__(self, num_pages: int):
        self.num_pages = int(num_pages)
        self.free: List[int] = list(range(self.num_pages - 1, -1, -1))  # pop() yields page 0 first
        self.holders: List[set] = [set() for _ in range(self.num_pages)]
        self.hash_of: List[Optional[int]] = [None] * self.num_pages     # prefix hash of a registered page
        self.key_of: List[Optional[tuple]] = [None] * self.num_pages    # (hash before the page, its tokens): told apart from a collision
        self.by_hash: Dict[int, int] = {}
        self.reclaimable: "OrderedDict[int, None]" = OrderedDict()      # registered, no holder; oldest first

    def alloc(self, owner: int) -> Optional[int]:
        if self.free:
            p = self.free.pop()
        elif self.reclaimable:
            p, _ = self.reclaimable.popitem(last=False)
            del self.by_hash[self.hash_of[p]]
            self.hash_of[p] = self.key_of[p] = None
        else:
            return None
        assert not self.holders[p], f"page {p} handed out while held by slots {sorted(self.holders[p])}"
        self.holders[p].add(owner)
        return p

    def release(self, page: int, owner: int) -> None:
        if owner not in self.holders[page]:
            raise MemoryError_(f"page {page} freed by slot {owner} but held by {sorted(self.holders[page])}")
        self.holders[page].discard(owner)
        if self.holders[page]:
            return
        if self.hash_of[page] is not None:
            self.reclaimable[page] = None
        else:
            self.free.append(page)

    def n_free(self) -> int:
        return len(self.free) + len(self.reclaimable)

    # ---- pages shared by their prefix ------------------------------------
    def register(self, page: int, h: int, key: tuple) -> None:
        """Make a full page findable under the hash ``h`` of the tokens up to its end; ``key`` =
        (hash before the page, the page's tokens) is kept to tell a match from a collision."""
        if self.hash_of[page] is None and h not in self.by_hash:
            self.hash_of[page] = h
            self.key_of[page] = key
            self.by_hash[h] = page

    def unregister(self, page: int) -> None:
        if self.hash_of[page] is not None:
            del self.by_hash[self.hash_of[page]]
            self.hash_of[page] = self.key_of[page] = None
            if page in self.reclaimable:
                del self.reclaimable[page]
                self.free.append(page)

    def lookup(self, h: int, key: tuple) -> Optional[int]:
        p = self.by_hash.get(h)
        return p if p is not None and self.key_of[p] == key else None

    def share(self, page: int, owner: int) -> None:
        """One more holder for a registered page."""
        assert self.hash_of[page] is not None
        self.reclaimable.pop(page, None)
        self.holders[page].add(owner)


@dataclass
class KVLayerView:
    """What a mixer sees of its cache: key pages, value pages, the group's table."""

    k_pages: torch.Tensor        # [num_pages, n_kv_heads, block_size, head_dim]
    v_pages: torch.Tensor
    block_table: torch.Tensor    # [max_slots, max_blocks] int32, NO_PAGE where none
    block_size: int
    window: Optional[int]
    group: int


@dataclass
class StateView:
    """Per-request state of fixed size: ``state[slot]`` belongs to the request in ``slot``."""

    state: torch.Tensor          # [max_slots, *shape]


class KVGroup:
    def __init__(self, index: int, spec: KVCacheSpec, block_size: int, num_pages: int, max_slots: int,
                 max_len: int):
        self.index = index
        self.spec = spec
        self.block_size = block_size
        self.window = spec.window
        self.max_blocks = -(-max_len // block_size)
        self.pool = PagePool(num_pages)
        self.entries: List[int] = []                   # run entries whose cache lives here
        self.table = np.full((max_slots, self.max_blocks), NO_PAGE, dtype=np.int32)
        self.n_blocks = [0] * max_slots                # logical blocks ever reached (high-water)
        self.first_live = [0] * max_slots              # lowest logical block not yet given back
        self.storage: Optional[torch.Tensor] = None    # [entries, 2, pages, kv heads, block, head_dim]
        self.table_dev: Optional[torch.Tensor] = None
        self.dirty: set = set()

    # -- arithmetic --------------------------------------------------------
    def _first_needed_block(self, next_query_pos: int) -> int:
        """Lowest logical block holding a key the query at ``next_query_pos`` may see."""
        if self.window is None:
            return 0
        return max(0, next_query_pos - self.window + 1) // self.block_size

    def pages_short(self, slot: int, start: int, new_len: int) -> int:
        """Pages to allocate so that positions start..new_len-1 can be written and read."""
        if new_len <= 0:
            return 0
        need_hi = -(-new_len // self.block_size)
        lo = max(self.n_blocks[slot], self._first_needed_block(start))
        return max(0, need_hi - lo)


class CacheManager:
    """Slots, groups, pools, tables and state arrays for one model."""

    def __init__(self, cache_needs: Sequence[Tuple[object, Optional[int]]], block_size: int, num_pages: int,
                 max_slots: int, max_len: int, dtype: torch.dtype, device, allocate: bool = True,
                 prefix_sharing: bool = False):
        if num_pages * block_size < 1:
            raise ConfigError("cache pool must hold at least one page")
        self.block_size = int(block_size)
        self.max_slots = int(max_slots)
        self.max_len = int(max_len)
        self.dtype = dtype
        self.device = torch.device(device) if allocate else None
        self.groups: List[KVGroup] = []
        self._group_of_entry: Dict[int, Tuple[int, int]] = {}   # run entry -> (group, index within group)
        self._state_entries: Dict[int, StateSpec] = {}
        self.state: Dict[int, torch.Tensor] = {}
        by_key: Dict[Tuple, KVGroup] = {}
        for ei, (spec, cache_of) in enumerate(cache_needs):
            if cache_of is not None or spec is None:
                continue
            if isinstance(spec, KVCacheSpec):
                key = (spec.n_kv_heads, spec.head_dim, spec.window)
                g = by_key.get(key)
                if g is None:
                    g = KVGroup(len(self.groups), spec, self.block_size, num_pages, max_slots, max_len)
                    by_key[key] = g
                    self.groups.append(g)
                self._group_of_entry[ei] = (g.index, len(g.entries))
                g.entries.append(ei)
            elif isinstance(spec, StateSpec):
                self._state_entries[ei] = spec
            else:
                raise ConfigError(f"run entry {ei}: unknown cache need {spec!r}")
        self.free_slots: List[int] = list(range(max_slots - 1, -1, -1))      # pop() yields slot 0 first
        self.live: List[bool] = [False] * max_slots
        self.length: List[int] = [0] * max_slots                             # positions cached per slot
        self.views: Dict[int, object] = {}
        # pages are shared by their token prefix only when every layer keeps all positions and no
        # mixer has state of its own: a prefix is then fully described by its pages
        self.prefix_sharing = bool(prefix_sharing) and not self._state_entries and \
            all(g.window is None for g in self.groups) and bool(self.groups)
        self._hashed: Dict[int, Tuple[int, int]] = {}   # slot -> (blocks hashed so far, hash of the last)
        self.prefix_hits = 0                 # positions taken over from registered pages
        self.prefix_misses = 0               # positions of prompts that had to be computed
        if allocate:
            self._allocate()

    # ------------------------------------------------------------------
    def _allocate(self):
        dev = self.device
        for g in self.groups:
            s = g.spec
            g.storage = torch.zeros((len(g.entries), 2, g.pool.num_pages, s.n_kv_heads, self.block_size, s.head_dim),
                                    dtype=self.dtype, device=dev)
            g.table_dev = torch.full((self.max_slots, g.max_blocks), NO_PAGE, dtype=torch.int32, device=dev)
            g.table_pinned = torch.from_numpy(g.table)
            if dev.type == "cuda":
                g.table_pinned = torch.full((self.max_slots, g.max_blocks), NO_PAGE, dtype=torch.int32).pin_memory()
                g.table = g.table_pinned.numpy()
            for j, ei in enumerate(g.entries):
                self.views[ei] = KVLayerView(g.storage[j, 0], g.storage[j, 1], g.table_dev, self.block_size,
                                             g.window, g.index)
        for ei, spec in self._state_entries.items():
            t = torch.zeros((self.max_slots, *spec.shape), dtype=getattr(torch, spec.dtype), device=dev)
            self.state[ei] = t
            self.views[ei] = StateView(t)

    def view(self, run_entry: int):
        return self.views.get(run_entry)

    # ---- slots -------------------------------------------------------
    def has_free_slot(self) -> bool:
        return bool(self.free_slots)

    def admit(self) -> Optional[int]:
        """Take a slot (None if all are in use); its state arrays start at zero."""
        if not self.free_slots:
            return None
        slot = self.free_slots.pop()
        assert not self.live[slot]
        self.live[slot] = True
        self.length[slot] = 0
        for g in self.groups:
            assert g.n_blocks[slot] == 0 and g.first_live[slot] == 0
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        """Give back every page the slot holds, then the slot itself."""
        if not self.live[slot]:
            raise MemoryError_(f"slot {slot} freed twice or never admitted")
        for g in self.groups:
            for b in range(g.first_live[slot], g.n_blocks[slot]):
                p = int(g.table[slot, b])
                if p != NO_PAGE:
                    g.pool.release(p, slot)
                    g.table[slot, b] = NO_PAGE
            g.n_blocks[slot] = 0
            g.first_live[slot] = 0
            g.dirty.add(slot)
        self.live[slot] = False
        self.length[slot] = 0
        self._hashed.pop(slot, None)
        self.free_slots.append(slot)

    # ---- queries for the scheduler -------------------------------------
    def free_pages(self) -> List[int]:
        return [g.pool.n_free() for g in self.groups]

    def pages_short(self, slot: Optional[int], new_len: int, start: Optional[int] = None) -> List[int]:
        """Per group: pages still to allocate for the slot to reach ``new_len`` positions
        (``slot`` None: a request not yet admitted)."""
        out = []
        for g in self.groups:
            if slot is None:
                out.append(-(-new_len // g.block_size) - g._first_needed_block(0 if start is None else start))
            else:
                out.append(g.pages_short(slot, self.length[slot] if start is None else start, new_len))
        return out

    def can_fit(self, demands: Sequence[Tuple[Optional[int], int]]) -> bool:
        """True if every group has pages for all of ``(slot or None, new_len)`` together."""
        total = [0] * len(self.groups)
        for slot, new_len in demands:
            for i, n in enumerate(self.pages_short(slot, new_len)):
                total[i] += n
        return all(t <= f for t, f in zip(total, self.free_pages()))

    # ---- growing and shrinking -------------------------------------------
    def ensure(self, slot: int, new_len: int) -> bool:
        """Allocate pages so positions length[slot]..new_len-1 can be written; all groups or none."""
        if not self.live[slot]:
            raise MemoryError_(f"slot {slot} is not live")
        if new_len > self.max_len:
            raise MemoryError_(f"slot {slot}: {new_len} positions exceed the maximum length {self.max_len}")
        start = self.length[slot]
        short = [g.pages_short(slot, start, new_len) for g in self.groups]
        if any(s > g.pool.n_free() for s, g in zip(short, self.groups)):
            return False
        for g in self.groups:
            need_hi = -(-new_len // g.block_size)
            lo = max(g.n_blocks[slot], g._first_needed_block(start))
            if lo > g.n_blocks[slot]:
                # blocks wholly outside the window are never allocated
                g.first_live[slot] = max(g.first_live[slot], lo)
            for b in range(lo, need_hi):
                p = g.pool.alloc(slot)
                assert p is not None
                g.table[slot, b] = p
            if need_hi > g.n_blocks[slot]:
                g.n_blocks[slot] = need_hi
                g.dirty.add(slot)
        return True

    def advance(self, slot: int, new_len: int) -> None:
        """Record that the slot now caches ``new_len`` positions; pages that the window of
        the next query has passed are given back."""
        self.length[slot] = new_len
        for g in self.groups:
            if g.window is None:
                continue
            keep_from = min(g._first_needed_block(new_len), g.n_blocks[slot])
            for b in range(g.first_live[slot], keep_from):
                p = int(g.table[slot, b])
                if p != NO_PAGE:
                    g.pool.release(p, slot)
                    g.table[slot, b] = NO_PAGE
                    g.dirty.add(slot)
            g.first_live[slot] = max(g.first_live[slot], keep_from)

    def truncate(self, slot: int, new_len: int) -> None:
        """Forget the positions from ``new_len`` on (the reference's ``truncate_to``,
        zllm src/backend/candle/backend.rs:95-114): pages wholly beyond them go back to their
        pools.  Refused when a windowed group has already given back pages that the next query at
        ``new_len`` would need, or when a mixer keeps per-request state (it cannot be rewound)."""
        if not self.live[slot]:
            raise MemoryError_(f"slot {slot} is not live")
        if not 0 <= new_len <= self.length[slot]:
            raise MemoryError_(f"slot {slot}: cannot truncate {self.length[slot]} positions to {new_len}")
        if new_len == self.length[slot]:
            return
        if new_len > 0:
            if self.state:
                raise MemoryError_("a model with per-request state cannot be truncated (only reset to 0)")
            for g in self.groups:
                if g._first_needed_block(new_len) < g.first_live[slot]:
                    raise MemoryError_(f"slot {slot}: the window's pages before position {new_len} were given back")
        if new_len % self.block_size:
            # the page that is kept partly will be written again: nobody else may rely on it
            b = new_len // self.block_size
            for g in self.groups:
                p = int(g.table[slot, b])
                if p != NO_PAGE and len(g.pool.holders[p]) > 1:
                    raise MemoryError_(f"slot {slot}: position {new_len} lies in a page shared with other requests")
            for g in self.groups:
                p = int(g.table[slot, b])
                if p != NO_PAGE:
                    g.pool.unregister(p)
        self._hashed.pop(slot, None)
        for g in self.groups:
            keep = -(-new_len // g.block_size)           # >= first_live when new_len > 0 (checked above)
            for b in range(max(keep, g.first_live[slot]), g.n_blocks[slot]):
                p = int(g.table[slot, b])
                if p != NO_PAGE:
                    g.pool.release(p, slot)
                    g.table[slot, b] = NO_PAGE
                    g.dirty.add(slot)
            g.n_blocks[slot] = min(g.n_blocks[slot], keep)
            if new_len == 0:
                g.first_live[slot] = 0
        if new_len == 0:
            for t in self.state.values():
                t[slot].zero_()
        self.length[slot] = new_len

    # ---- pages shared by their token prefix (mod.rs:1941-1947,2276-2317) --------------
    def _next_hash(self, h: int, tokens: Sequence[int], b: int):
        """(hash of the tokens up to the end of block b, the key that confirms a match)."""
        bs = self.block_size
        key = (h, tuple(tokens[b * bs:(b + 1) * bs]))
        return hash(key), key

    def adopt_prefix(self, slot: int, tokens: Sequence[int]) -> int:
        """For a slot that holds nothing yet: take over the longest run of registered pages whose
        chained hashes match the full blocks of ``tokens`` -- never the block with the last token,
        so that at least one position is left to compute.  Returns the positions taken over
        (the slot's cached length afterwards)."""
        if not self.prefix_sharing or not self.live[slot] or self.length[slot] != 0 or \
                any(g.n_blocks[slot] for g in self.groups):
            return 0
        max_reuse = (len(tokens) - 1) // self.block_size
        h, run = 0, []
        for b in range(max_reuse):
            h, key = self._next_hash(h, tokens, b)
            pages = [g.pool.lookup(h, key) for g in self.groups]
            if any(p is None for p in pages):
                break
            run.append((h, pages))
        for b, (_, pages) in enumerate(run):
            for g, p in zip(self.groups, pages):
                g.pool.share(p, slot)
                g.table[slot, b] = p
        n = len(run)
        if n:
            for g in self.groups:
                g.n_blocks[slot] = n
                g.dirty.add(slot)
            self._hashed[slot] = (n, run[-1][0])
        self.length[slot] = n * self.block_size
        self.prefix_hits += n * self.block_size
        self.prefix_misses += len(tokens) - n * self.block_size
        return n * self.block_size

    def register_prefix(self, slot: int, tokens: Sequence[int], upto: int) -> None:
        """The slot's full pages below position ``upto`` (all written) become findable by the hash
        of the tokens up to their end."""
        if not self.prefix_sharing:
            return
        nb = min(upto, len(tokens), self.length[slot]) // self.block_size
        done, h = self._hashed.get(slot, (0, 0))
        for b in range(done, nb):
            h, key = self._next_hash(h, tokens, b)
            for g in self.groups:
                g.pool.register(int(g.table[slot, b]), h, key)
        if nb > done:
            self._hashed[slot] = (nb, h)

    table_bytes_uploaded = 0        # host-to-device bytes of block-table rows so far (for measurement)

    def sync_tables(self) -> None:
        """Copy the table rows that changed since the last call to the device."""
        for g in self.groups:
            if g.table_dev is None:
                g.dirty.clear()
                continue
            for slot in sorted(g.dirty):
                g.table_dev[slot].copy_(g.table_pinned[slot], non_blocking=True)
                self.table_bytes_uploaded += g.table_pinned[slot].numel() * 4
            g.dirty.clear()

    # ---- integrity ------------------------------------------------------
    def check_integrity(self) -> None:
        """No page lost, held by a slot that does not list it, free or reclaimable while held,
        shared without being registered; raises AssertionError otherwise."""
        for g in self.groups:
            held: Dict[int, set] = {}
            for slot in range(self.max_slots):
                row = g.table[slot]
                pages = [int(p) for p in row if p != NO_PAGE]
                if not self.live[slot]:
                    assert not pages, f"group {g.index}: dead slot {slot} holds pages {pages}"
                assert len(set(pages)) == len(pages), f"group {g.index}: slot {slot} lists a page twice"
                for b, p in enumerate(row):
                    if p == NO_PAGE:
                        continue
                    assert g.first_live[slot] <= b < g.n_blocks[slot], f"page outside live range in slot {slot}"
                    held.setdefault(int(p), set()).add(slot)
            pool = g.pool
            for p in range(pool.num_pages):
                assert pool.holders[p] == held.get(p, set()), (
                    f"group {g.index}: page {p} held by {sorted(pool.holders[p])} but listed by {sorted(held.get(p, set()))}")
                if len(pool.holders[p]) > 1:
                    assert pool.hash_of[p] is not None, f"group {g.index}: page {p} is shared but not registered"
                if pool.hash_of[p] is not None:
                    assert pool.by_hash.get(pool.hash_of[p]) == p
            free, rec = pool.free, list(pool.reclaimable)
            assert len(set(free)) == len(free), f"group {g.index}: a page is on the free stack twice"
            assert not (set(free) & set(held)) and not (set(rec) & set(held)), f"group {g.index}: a held page is free"
            assert not (set(free) & set(rec))
            assert all(pool.hash_of[p] is not None for p in rec) and all(pool.hash_of[p] is None for p in free)
            assert len(pool.by_hash) == sum(h is not None for h in pool.hash_of)
            assert len(free) + len(rec) + len(held) == pool.num_pages, (
                f"group {g.index}: {pool.num_pages - len(free) - len(rec) - len(held)} pages lost")
        assert len(set(self.free_slots)) == len(self.free_slots)
        assert sum(self.live) + len(self.free_slots) == self.max_slots
