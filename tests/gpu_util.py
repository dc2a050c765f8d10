"""Helpers of the GPU tests: a small step description and cache made by hand."""
from __future__ import annotations

import torch

from zllm_b200.cache import CacheManager
from zllm_b200.engine.batch import StepBuffers, StepEntry, Workspace, fill_step, make_context
from zllm_b200.parts import KVCacheSpec

DEV = "cuda:0"

# bf16 has 8 bits of mantissa: one rounding is 2^-9 relative.  Whole-model logits pass through
# ~10 roundings per layer.  The bound of a comparison is a fraction of the request's largest
# |logit|, per configuration: twice the worst error observed on a B200 over the whole suite
# (every observation is recorded by ``observe`` and printed at the end of a run), so that a
# fault that doubles the error of a single position shows.  BF16_MAX_OF_SCALE is the ceiling
# that no configuration may exceed and the bound of configurations without an entry.
BF16_MAX_OF_SCALE = 0.04
# observed over the suite at the configurations' own weight scales: A 0.0017, B 0.0067, C 0.0071,
# D 0.0075, E 0.0064, the 1B layer sizes 0.0096
BF16_OF_SCALE = {"A": 0.0035, "B": 0.0135, "C": 0.0145, "D": 0.015, "E": 0.013, "1B layers": 0.02}
# Token streams at the sharper weights of ``configs.GEN_STD``: a greedy choice may flip when the
# two best plain logits are closer than the sum of their errors.  The largest gap of a flipped
# choice observed over the suite is 0.9 % of the largest logit; twice that counts as a near-tie.
BF16_GAP_OF_SCALE = 0.02
F32_ATOL = 1e-4

OBSERVED = {}            # what -> (worst error / scale, bound / scale)


def bf16_bound(name=None):
    """The bfloat16 bound, as a fraction of the largest |logit|, of tiny configuration ``name``."""
    return min(BF16_OF_SCALE.get(name, BF16_MAX_OF_SCALE), BF16_MAX_OF_SCALE)


def observe(what, err, scale, bound_of_scale):
    """Record the worst error seen under the label ``what`` (printed at the end of the run)."""
    frac = err / scale if scale > 0 else 0.0
    old = OBSERVED.get(what)
    if old is None or frac > old[0]:
        OBSERVED[what] = (frac, bound_of_scale)


def check_greedy_stream(forward, prompt, got, dtype, max_tokens, stop=(), gap_of_scale=None, what="stream"):
    """A greedy stream against the plain implementation, teacher-forced on the stream itself:
    ``forward(tokens)`` gives the plain logits [T, V] of a whole sequence.  Every produced token
    must be the plain argmax given the stream so far; in bfloat16 it may instead be a token
    whose plain logit lies within ``gap_of_scale`` of the largest (a near-tie that rounding may
    flip).  The stream must end exactly at its first stop token or at ``max_tokens``."""
    assert len(got) >= 1, f"{what}: nothing was produced"
    if any(t in stop for t in got):
        k = next(i for i, t in enumerate(got) if t in stop)
        assert len(got) == k + 1, f"{what}: {len(got) - k - 1} tokens after the stop token at {k}"
    else:
        assert len(got) == max_tokens, f"{what}: {len(got)} tokens, expected {max_tokens}"
    lg = forward(list(prompt) + list(got[:-1]))[len(prompt) - 1:]
    for i, t in enumerate(got):
        row = lg[i]
        best = int((row == row.max()).nonzero()[0])
        if t == best:
            continue
        assert dtype != "float32", f"{what}: token {i} is {t}, plain says {best}"
        gap = float(row[best] - row[t])
        scale = float(row.abs().max())
        lim = (gap_of_scale if gap_of_scale is not None else BF16_GAP_OF_SCALE) * scale
        observe(f"near-tie gap {what}", gap, scale, lim / scale)
        assert gap <= lim, f"{what}: token {i} is {t} (plain {best}), gap {gap:.3e} > {lim:.3e}"


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
    from zllm_b200.kernels.ops import CudaOps
    T, R, nd, plans, mc = fill_step(buf, ents, starts, planners=(CudaOps.plan_query_tiles,))
    buf.upload()
    cm.sync_tables()
    ctx = make_context(buf, T, R, nd, plans, mc, Workspace(max_rows, DEV), ents, starts)
    for (slot, n), s in zip(entries, starts):
        cm.advance(slot, s + n)
    return ctx


def cpu_ctx(ctx):
    """The same description with its arrays on the CPU (for the plain statements)."""
    import copy
    c = copy.copy(ctx)
    for k in ("token_ids", "positions", "row_slot", "want_rows", "decode_rows"):
        setattr(c, k, getattr(ctx, k).cpu())
    c.aux = {k: v.cpu() for k, v in ctx.aux.items()}
    return c


class CpuCacheView:
    def __init__(self, view):
        self.k_pages = view.k_pages.float().cpu()
        self.v_pages = view.v_pages.float().cpu()
        self.block_table = view.block_table.cpu()
        self.block_size = view.block_size
        self.window = view.window
