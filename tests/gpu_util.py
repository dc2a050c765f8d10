"""Helpers of the GPU tests: a small step description and cache made by hand."""
from __future__ import annotations

import torch

from zllm_b200.cache import CacheManager
from zllm_b200.engine.batch import StepBuffers, StepEntry, Workspace, fill_step, make_context
from zllm_b200.parts import KVCacheSpec

DEV = "cuda:0"

# bf16 has 8 bits of mantissa: one rounding is 2^-9 relative.  Whole-model logits pass through
# ~10 roundings per layer; the bound below (of the largest |logit|) is fixed, not fitted.
BF16_MAX_OF_SCALE = 0.04
F32_ATOL = 1e-4


def make_cache(nkv, hd, bs, pages, slots, max_len, dtype, window=None, layers=1):
    needs = [(KVCacheSpec(nkv, hd, window), None)] * layers
    return CacheManager(needs, bs, pages, slots, max_len, dtype, DEV)


def make_ctx(cm, entries, max_rows=4096):
    """entries: [(slot, n_tokens)] appended at each slot's cached length; pages are ensured."""
    buf = StepBuffers(max_rows, max_rows, DEV)
    ents, starts = [], []
    for slot, n in entries:
        start = cm.length[slot]
        assert cm.ensure(slot, start + n)
        ents.append(StepEntry(slot, [0] * n, ()))
        starts.append(start)
    T, R, nd, nt, mc = fill_step(buf, ents, starts)
    buf.upload()
    cm.sync_tables()
    ctx = make_context(buf, T, R, nd, nt, mc, Workspace(max_rows, DEV), ents, starts)
    for (slot, n), s in zip(entries, starts):
        cm.advance(slot, s + n)
    return ctx


def cpu_ctx(ctx):
    """The same description with its arrays on the CPU (for the plain statements)."""
    import copy
    c = copy.copy(ctx)
    for k in ("token_ids", "positions", "row_slot", "want_rows", "decode_rows", "tiles"):
        setattr(c, k, getattr(ctx, k).cpu())
    return c


class CpuCacheView:
    def __init__(self, view):
        self.k_pages = view.k_pages.float().cpu()
        self.v_pages = view.v_pages.float().cpu()
        self.block_table = view.block_table.cpu()
        self.block_size = view.block_size
        self.window = view.window
