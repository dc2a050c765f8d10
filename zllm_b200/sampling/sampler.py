"""Turning a step's logits into tokens.

Three ways, after the reference (zllm src/backend/gpu/batch.rs:184-194 picks
"the cheapest path that satisfies every active stream"):

* greedy and plain temperature: one kernel per step samples every row on the
  device (argmax, or Gumbel-max with the counter-based noise of
  src/backend/gpu/shaders.rs:796-850); only token ids come back.
* top-k / top-p: the device extracts each row's 64 best logits (BTOPK,
  shaders.rs:852-905) and the draw among them with splitmix64
  (src/backend/gpu/sampling.rs:24-56) is made either on the host (``sample_from_pool``
  below: mixed steps, engines without CUDA graphs) or, in double precision and with the
  same arithmetic, by a kernel inside the captured decode step (csrc/sampling.cu,
  ``ModelRunner.decode_step(pool=...)``), so that such requests decode without the host
  between steps like greedy ones.
* min-p, or top-k beyond the pool: the row's logits come to the host and the full
  chain temperature -> top-k -> softmax -> min-p -> top-p -> inverse-CDF draw of
  src/engine/sampler.rs:31-128 runs there.

The reference applies top-k/top-p only from the second generated token on
(batch.rs:133-135, a limit of its prefill path); here they apply to every token.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import torch

from .params import SamplingParams, TOPK_POOL, step_seed

_M64 = (1 << 64) - 1


def rng01(seed: int) -> float:
    """Uniform in (0,1) from a 32-bit seed by splitmix64 (sampling.rs:24-30)."""
    z = ((seed & 0xFFFFFFFF) * 0x9E3779B97F4A7C15 + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return ((z >> 40) + 0.5) / 16777216.0


def sample_from_pool(vals: Sequence[float], idxs: Sequence[int], p: SamplingParams, seed: int) -> int:
    """Draw among descending candidates (sampling.rs:35-56)."""
    n = 0
    for v in vals:
        if v > -3.0e37:
            n += 1
        else:
            break
    n = min(n, len(idxs))
    if n == 0 or p.is_greedy:
        return int(idxs[0])
    kk = n if p.top_k == 0 else min(p.top_k, n)
    mx = vals[0]
    probs = [math.exp((vals[i] - mx) / p.temperature) for i in range(kk)]
    z = sum(probs)
    probs = [q / z for q in probs]
    cut = kk
    if 0.0 < p.top_p < 1.0:
        cum = 0.0
        for i, q in enumerate(probs):
            cum += q
            if cum >= p.top_p:
                cut = i + 1
                break
    zc = sum(probs[:cut])
    target = rng01(seed) * zc
    acc = 0.0
    for i in range(cut):
        acc += probs[i]
        if acc >= target:
            return int(idxs[i])
    return int(idxs[cut - 1])


def sample_full(logits: torch.Tensor, p: SamplingParams, seed: int) -> int:
    """The whole-vocabulary chain of sampler.rs:31-128 on the host, drawn with ``rng01(seed)``."""
    lg = logits.detach().float().cpu()
    if p.is_greedy:
        mx = lg.max()
        return int((lg == mx).nonzero()[0])
    if p.temperature != 1.0:
        lg = lg / p.temperature
    V = lg.numel()
    if 0 < p.top_k < V:
        thr = torch.sort(lg, descending=True, stable=True).values[p.top_k - 1]
        lg = torch.where(lg < thr, torch.tensor(float("-inf")), lg)
    probs = torch.softmax(lg, dim=-1)
    if p.min_p > 0.0:
        cutoff = p.min_p * probs.max()
        probs = torch.where(probs < cutoff, torch.zeros(()), probs)
        kept = probs.sum()
        if kept > 0:
            probs = probs / kept
    if p.top_p < 1.0:
        sp, si = torch.sort(probs, descending=True, stable=True)
        cum = torch.cumsum(sp, 0) - sp          # mass before each candidate
        keep = cum < p.top_p                    # "if cumsum >= top_p: break" before adding
        filt = torch.zeros_like(probs)
        filt[si[keep]] = sp[keep]
        s = filt.sum()
        if s > 0:
            probs = filt / s
    r = rng01(seed)
    cdf = torch.cumsum(probs, 0)
    hit = (cdf >= r).nonzero()
    return int(hit[0]) if hit.numel() else V - 1


class Sampler:
    """Samples the wanted rows of a step.  ``ops`` is the kernel table."""

    def __init__(self, ops, device, max_rows: int):
        self.ops = ops
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.temps = torch.zeros(max_rows, dtype=torch.float32, device=self.device)
        self.seeds = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self.out = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self.pool_vals = torch.zeros((max_rows, TOPK_POOL), dtype=torch.float32, device=self.device)
        self.pool_idx = torch.zeros((max_rows, TOPK_POOL), dtype=torch.int32, device=self.device)

    def host_finish(self, logits: torch.Tensor, device_tokens: Sequence[int], params: Sequence[SamplingParams],
                    seeds: Sequence[int]) -> List[int]:
        """Replace the device's tokens for rows that need the pool or the full chain."""
        out = [int(t) for t in device_tokens]
        R = len(params)
        if any(p.needs_topk and not p.needs_full for p in params):
            k = min(TOPK_POOL, logits.shape[1])
            vals = self.pool_vals[:R, :k].contiguous() if k != TOPK_POOL else self.pool_vals[:R]
            idx = self.pool_idx[:R, :k].contiguous() if k != TOPK_POOL else self.pool_idx[:R]
            self.ops.topk(logits[:R], k, vals, idx)
            hv, hi = vals.cpu().tolist(), idx.cpu().tolist()
            for r, p in enumerate(params):
                if p.needs_topk and not p.needs_full:
                    out[r] = sample_from_pool(hv[r], hi[r], p, seeds[r])
        for r, p in enumerate(params):
            if p.needs_full:
                out[r] = sample_full(logits[r], p, seeds[r])
        return out

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int]) -> List[int]:
        """logits [R, V] float32 on the device; one token per row."""
        R = len(params)
        t = torch.tensor([0.0 if (p.is_greedy or p.needs_topk or p.needs_full) else p.temperature for p in params],
                         dtype=torch.float32)
        s = torch.tensor([x & 0xFFFFFFFF for x in seeds], dtype=torch.int64).to(torch.int32)
        self.temps[:R].copy_(t)
        self.seeds[:R].copy_(s)
        self.ops.sample(logits[:R], self.temps[:R], self.seeds[:R], self.out[:R])
        toks = self.out[:R].cpu().tolist()
        check = getattr(self.ops, "raise_if_a_wait_gave_up", None)
        if check is not None:
            check()                 # the copy above waited for the step: a wait that ran out has flagged it
        return self.host_finish(logits, toks, params, seeds)
