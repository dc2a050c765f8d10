"""The description of one step's batch, as the kernels read it.

The reference's step takes parallel arrays ``tokens[m], positions[m], slots[m]``;
rows of one slot at consecutive positions are a prompt portion, and causality
inside a portion comes from the positions alone because every row's key and
value are written before any row attends (zllm src/backend/gpu/mod.rs:2165,
2245-2253, 2485-2491).  The same here, plus which rows are single decoded
tokens.  What a particular kernel wants beyond that (the attention kernels'
query tiles, say) is not described here: a part may register a *planner* that
writes its own integer tables into the step buffer's auxiliary region, which
goes to the device with the same single copy.

All integer arrays of a step live in ONE pinned host buffer and ONE device
buffer with fixed section offsets, so a step costs one host-to-device copy and
a captured graph can be replayed on new contents.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

@dataclass
class StepEntry:
    """One request's share of a step: its slot, its next tokens, and the places among
    them whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepBuffers:
    """Pinned host + device int32 storage for a step of at most ``cap_rows`` rows."""

    # the two float64 sections come first so that they are 8-byte aligned
    SECTIONS = ("pool_temp", "pool_topp", "token_ids", "positions", "row_slot", "want_rows", "decode_rows", "aux", "temps",
                "seeds", "pool_topk")

    def __init__(self, cap_rows: int, cap_want: int, device):
        self.cap_rows = cap_rows
        self.cap_want = cap_want
        sizes = {"token_ids": cap_rows, "positions": cap_rows, "row_slot": cap_rows, "want_rows": cap_want,
                 # the parts' own tables of a step (see ``AuxRegion``)
                 "decode_rows": cap_rows, "aux": 4 * cap_rows + 64, "temps": cap_want, "seeds": cap_want,
                 # candidate-pool sampling of a wanted row: temperature and top_p as float64 (two words), top_k
                 "pool_temp": 2 * cap_want, "pool_topp": 2 * cap_want, "pool_topk": cap_want}
        self.offsets = {}
        off = 0
        for name in self.SECTIONS:
            self.offsets[name] = (off, sizes[name])
            off += sizes[name]
        self.total = off
        dev = torch.device(device)
        self.host = torch.zeros(off, dtype=torch.int32)
        if dev.type == "cuda":
            self.host = self.host.pin_memory()
        self.np = self.host.numpy()
        self.dev = torch.zeros(off, dtype=torch.int32, device=dev)
        self.copied = torch.cuda.Event() if dev.type == "cuda" else None
        self._pending = False

    @staticmethod
    def table_shapes(entries, starts, planners):
        """The names and (bucketed) shapes of the tables the planners would make for this step,
        without a buffer: what a step graph's key needs."""
        if not planners:
            return ()
        scratch = AuxRegion(np.zeros(4 * sum(len(e.tokens) for e in entries) + 64, dtype=np.int32))
        out = []
        for plan in planners:
            out.extend((name, tuple(shape)) for name, (_, shape) in plan(entries, starts, scratch, bucketed=True).items())
        return tuple(sorted(out))

    def host_section(self, name):
        o, n = self.offsets[name]
        return self.np[o:o + n]

    def dev_section(self, name, n=None):
        o, size = self.offsets[name]
        return self.dev[o:o + (size if n is None else n)]

    def begin_fill(self):
        if self._pending and self.copied is not None:
            self.copied.synchronize()   # the previous copy must have read the pinned buffer
            self._pending = False

    bytes_uploaded = 0          # host-to-device bytes of all step buffers so far (for measurement)

    def upload(self):
        StepBuffers.bytes_uploaded += self.total * 4
        self.dev.copy_(self.host, non_blocking=True)
        if self.copied is not None:
            self.copied.record()
            self._pending = True


class AuxRegion:
    """Hands out pieces of the step buffer's auxiliary section to the planners of a step.
    ``take(n)`` returns (host int32 view of n words, its offset in the section)."""

    def __init__(self, host_view):
        self.host = host_view
        self.used = 0

    def take(self, n: int):
        if self.used + n > self.host.shape[0]:
            raise MemoryError(f"the step buffer's auxiliary region holds {self.host.shape[0]} words; "
                              f"{self.used + n} were asked for")
        off = self.used
        self.used += n
        return self.host[off:off + n], off


@dataclass
class StepContext:
    """What parts and kernels see of a step."""

    T: int                       # rows in this step (for a replayed graph: the bucket size)
    R: int                       # rows whose logits are wanted
    token_ids: torch.Tensor      # [T] int32
    positions: torch.Tensor      # [T] int32 absolute position of each row
    row_slot: torch.Tensor       # [T] int32 slot of each row (-1: padding row, skipped)
    want_rows: torch.Tensor      # [R] int32
    decode_rows: torch.Tensor    # [n_decode] int32 rows that are single decoded tokens
    n_decode: int
    aux: dict                    # name -> int32 device table a part's planner wrote for this step
    max_context: int             # largest position + 1 among the rows (bounds split counts)
    ws: object = None            # workspace
    entries: Optional[List[StepEntry]] = None
    starts: Optional[List[int]] = None
    fixed_splits: int = 0        # > 0: the split count a captured graph was recorded with


def fill_step(buf: StepBuffers, entries: Sequence[StepEntry], starts: Sequence[int], pad_rows: int = 0, planners=(),
              pad_decode: Optional[int] = None, pad_want: int = 0, bucketed: bool = False):
    """Write the step's arrays into ``buf`` (host side) and return the counts
    (rows, wanted rows, decoded rows, the planners' tables, largest context).

    ``starts[i]`` is the position of entry i's first token.  ``pad_rows`` > 0
    pads the row arrays to that many rows with slot -1 (for graph buckets).
    ``planners``: callables ``(entries, starts, aux: AuxRegion) -> {name: (offset, shape)}`` of
    the model's parts; each writes what its kernels want to know about this step.
    For steps replayed from a captured graph every count must be that of the graph: ``pad_decode``
    pads the list of decoded rows to that many with padding rows (default: every padding row is
    one), ``pad_want`` the wanted rows with row 0, and ``bucketed`` asks the planners to round
    their tables up to sizes of their own choosing (``bucketed=True`` in their call).
    """
    buf.begin_fill()
    tok = buf.host_section("token_ids")
    pos = buf.host_section("positions")
    rs = buf.host_section("row_slot")
    want = buf.host_section("want_rows")
    dec = buf.host_section("decode_rows")
    r = 0
    nw = 0
    nd = 0
    max_ctx = 0
    for e, start in zip(entries, starts):
        n = len(e.tokens)
        tok[r:r + n] = e.tokens
        pos[r:r + n] = np.arange(start, start + n, dtype=np.int32)
        rs[r:r + n] = e.slot
        for w in e.want:
            if not 0 <= w < n:
                raise IndexError(f"wanted place {w} outside the entry's {n} tokens")
            want[nw] = r + w
            nw += 1
        if n == 1:
            dec[nd] = r
            nd += 1
        max_ctx = max(max_ctx, start + n)
        r += n
    T = r
    if pad_rows > T:
        tok[T:pad_rows] = 0
        pos[T:pad_rows] = 0
        rs[T:pad_rows] = -1
        more = pad_rows - T if pad_decode is None else max(0, pad_decode - nd)
        if more > pad_rows - T:
            raise ValueError("not enough padding rows for the decoded rows of the bucket")
        for i in range(T, T + more):
            dec[nd] = i
            nd += 1
        T = pad_rows
    if pad_want > nw:
        want[nw:pad_want] = 0
        nw = pad_want
    plans = {}
    if planners:
        aux = AuxRegion(buf.host_section("aux"))
        for plan in planners:
            plans.update(plan(entries, starts, aux, bucketed=True) if bucketed else plan(entries, starts, aux))
    return T, nw, nd, plans, max_ctx


def make_context(buf: StepBuffers, T, R, nd, plans, max_ctx, ws, entries=None, starts=None) -> StepContext:
    aux_dev = buf.dev_section("aux")
    aux = {}
    for name, (off, shape) in (plans or {}).items():
        n = 1
        for d in shape:
            n *= d
        aux[name] = aux_dev[off:off + n].view(*shape)
    return StepContext(
        T=T, R=R,
        token_ids=buf.dev_section("token_ids", T),
        positions=buf.dev_section("positions", T),
        row_slot=buf.dev_section("row_slot", T),
        want_rows=buf.dev_section("want_rows", R),
        decode_rows=buf.dev_section("decode_rows", nd),
        n_decode=nd,
        aux=aux,
        max_context=max_ctx,
        ws=ws, entries=list(entries) if entries is not None else None, starts=list(starts) if starts else None,
    )


class Workspace:
    """Named scratch buffers, allocated once at their largest first dimension.

    A buffer that has to grow is REPLACED, and the old one is kept for the workspace's life:
    captured CUDA graphs hold the addresses of the buffers they were captured with, and memory
    given back to the allocator would be handed to someone else while those graphs still write it.
    """

    def __init__(self, max_rows: int, device):
        self.max_rows = max_rows
        self.device = torch.device(device)
        self._bufs = {}
        self._retired = []
        self._views = {}                # (name, shape, dtype) -> the view handed out last time

    def get(self, name: str, shape, dtype, cap=None) -> torch.Tensor:
        """A [rows, ...] view of the buffer ``name``.  The buffer is made for ``cap`` rows
        (default: the step's row limit) the first time and only ever grows."""
        vkey = (name, shape, dtype) if type(shape) is tuple else (name, tuple(shape), dtype)
        view = self._views.get(vkey)
        if view is not None:            # a step asks for the same few views layer after layer
            return view
        rows = shape[0]
        rest = tuple(shape[1:])
        key = (name, rest, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[0] < rows:
            cap = max(rows, self.max_rows if cap is None else cap)
            if buf is not None:
                self._retired.append(buf)
                self._views = {k: v for k, v in self._views.items() if (k[0], tuple(k[1][1:]), k[2]) != key}
            buf = torch.empty((cap, *rest), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        if len(self._views) > 4096:     # many distinct row counts over a long run: start over
            self._views.clear()
        view = self._views[vkey] = buf[:rows]
        return view

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in list(self._bufs.values()) + self._retired)
