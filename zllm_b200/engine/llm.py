"""The Python entry point: an engine that takes token-id prompts to generated
token ids, in the manner of the reference's library calls.

zllm's callers use ``ContinuousBatcher::{enqueue_params(id, prompt, max_tokens,
eos, params, seed), step() -> Vec<(id, token, done)>, cancel(id)}``
(src/backend/gpu/batch.rs:64-211) and, single-stream, ``CandleCpuBackend::
{load_model, forward_logits(&[u32]) -> Vec<f32>, generate_token, reset_position,
truncate_to}`` (src/backend/candle/backend.rs:53-328).  ``Engine`` offers the
first set (``add_request`` / ``step`` / ``cancel`` / ``generate``) and ``Session``
the second, both over the same model, cache, step function and kernels.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import torch

from ..config.engine_config import EngineConfig
from ..errors import RequestError
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Plan, Scheduler


def _step_log():
    """ZLLM_STEP_LOG=path (or "-" for stderr): one JSON line per engine step -- what it ran, the
    wall time since the step before, queue lengths, free pages, and with ZLLM_PROFILE=1 the device
    time per kernel class.  The reference prints per-section timers from its ``profile`` feature
    (zllm src/main.rs:643-658); this is the same aid for a batched engine."""
    import os
    import sys
    import time
    path = os.environ.get("ZLLM_STEP_LOG")
    if not path:
        return None
    return {"f": sys.stderr if path == "-" else open(path, "a"), "t": time.perf_counter()}


class Engine:
    """Continuous batching over one model on one GPU.

    ``Engine(model_dir)`` loads a folder with config.json and model.safetensors;
    ``Engine(config=cfg, seed=s)`` makes random weights for a typed configuration.
    Keyword arguments are the fields of ``EngineConfig``.
    """

    def __init__(self, model: Optional[str] = None, *, config=None, seed: Optional[int] = None, ops=None,
                 engine_config: Optional[EngineConfig] = None, random_on_device: bool = False, **kw):
        ecfg = engine_config or EngineConfig(**kw)
        self.runner = ModelRunner(model, config=config, seed=seed, engine_config=ecfg, ops=ops,
                                  random_on_device=random_on_device)
        self.config = self.runner.config
        self.scheduler = Scheduler(self.runner.cache, ecfg.max_num_batched_tokens, self.runner.max_len)
        self.sampler = Sampler(self.runner.ops, self.runner.device, max(ecfg.max_num_seqs, 1))
        self.steps = 0
        self.generated = 0
        # what the last ``step()`` ran: decoded rows, prompt tokens, and whether it was a decode
        # graph launched ahead of the host (for measurement and the per-step log)
        self.last_step = {"decodes": 0, "prompt_tokens": 0, "ahead": False}
        self._log = _step_log()
        self.overlap = True            # launch the next decode step before reading this one's tokens
        self._ahead = None             # (requests, handle) of a decode step launched ahead
        # top-k / top-p draws inside the decode graph (no host between steps); off: the host draws
        self._device_pool = bool(self.runner.ecfg.cuda_graphs and self.runner.device.type == "cuda" and hasattr(self.runner.ops, "pool_draw"))

    # ---- requests ------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[int] = None) -> int:
        V = self.runner.spec.vocab_size
        for t in prompt_token_ids:
            if not 0 <= int(t) < V:
                raise RequestError(f"token id {t} is outside the vocabulary of {V}")
        return self.scheduler.add(prompt_token_ids, params or SamplingParams.greedy(), request_id)

    def cancel(self, request_id: int) -> bool:
        return self.scheduler.cancel(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # ---- one step ----------------------------------------------------------
    def _can_run_ahead(self, reqs, uncommitted: int) -> bool:
        """May the step after the one in flight be launched before its tokens are known?  Only in
        the steady state of decoding: nothing to admit or prefill, the same requests, sampling on
        the device, and none of them ends by length at the step in flight."""
        sch = self.scheduler
        if not self.overlap or sch.waiting or sch.prefilling or sch.preempted or len(reqs) != len(sch.running) \
                or any(a is not b for a, b in zip(reqs, sch.running)):
            return False
        for r in reqs:
            p = r.params
            if p.needs_full or (p.needs_topk and not self._device_pool) or r.gen_index + uncommitted >= p.max_tokens \
                    or len(r.tokens) + uncommitted + 1 >= self.runner.max_len:
                return False
        return True

    def _commit_ahead(self, reqs, toks):
        """Commit a step that was launched ahead: rows of requests that ended meanwhile (a stop
        token in the step before, a cancel) are dropped."""
        from .scheduler import RUNNING
        live = [(r, t) for r, t in zip(reqs, toks) if r.state == RUNNING]
        plan = Plan(decodes=[r for r, _ in live])
        out = self.scheduler.commit(plan, [t for _, t in live], [])
        self.steps += 1
        self.generated += len(out)
        return out

    def step(self):
        """One scheduler step: [(request id, token, done)] for every token produced.

        While only decoding, the step after the one whose tokens are being returned is already
        running on the device when this call returns (its inputs were advanced on the device), so
        the host's share of a step overlaps the device's.  A request that ends on a stop token
        has then computed one token too many, which is dropped."""
        if self._ahead is not None:
            reqs, handle = self._ahead
            self._ahead = None
            nxt = self.runner.decode_continue(handle) if self._can_run_ahead(reqs, 1) else None
            out = self._commit_ahead(reqs, self.runner.decode_collect(handle))
            if nxt is not None:
                self._ahead = (reqs, nxt)
            self._note(len(reqs), 0, True, out)
            return out
        plan = self.scheduler.schedule()
        if plan.empty:
            return []
        dec = plan.decodes
        dparams = [r.params for r in dec]
        dseeds = [r.next_seed() for r in dec]
        first: List[Optional[int]] = [None] * len(plan.portions)
        if not plan.portions:
            temps = [0.0 if (p.is_greedy or p.needs_topk or p.needs_full) else p.temperature for p in dparams]
            # top-k / top-p rows are drawn among their 64 best candidates on the device when decode
            # steps are graphs and no row needs the whole-vocabulary chain on the host
            on_device = self._device_pool and any(p.needs_topk for p in dparams) and not any(p.needs_full for p in dparams)
            pool = None
            if on_device:
                pool = ([p.temperature if p.needs_topk else 0.0 for p in dparams], [p.top_k for p in dparams],
                        [p.top_p for p in dparams])
            handle = self.runner.decode_launch([r.slot for r in dec], [r.tokens[-1] for r in dec], temps, dseeds, pool)
            nxt = self.runner.decode_continue(handle) if self._can_run_ahead(dec, 1) else None
            toks = self.runner.decode_collect(handle)
            if nxt is not None:
                self._ahead = (list(dec), nxt)
            if not on_device and any(p.needs_topk or p.needs_full for p in dparams):
                toks = self.sampler.host_finish(self.runner.last_logits, toks, dparams, dseeds)
            dtoks = toks
        else:
            entries = [StepEntry(r.slot, (r.tokens[-1],), (0,)) for r in dec]
            params, seeds = list(dparams), list(dseeds)
            for p in plan.portions:
                r = p.request
                entries.append(StepEntry(r.slot, r.tokens[p.start:p.start + p.n], (p.n - 1,) if p.completes else ()))
                if p.completes:
                    params.append(r.params)
                    seeds.append(r.next_seed())
            logits = self.runner.step(entries)
            toks = self.sampler.sample(logits, params, seeds) if params else []
            dtoks = toks[:len(dec)]
            rest = iter(toks[len(dec):])
            first = [next(rest) if p.completes else None for p in plan.portions]
        out = self.scheduler.commit(plan, dtoks, first)
        self.steps += 1
        self.generated += len(out)
        self._note(len(dec), sum(p.n for p in plan.portions), False, out)
        return out

    def _note(self, decodes, prompt_tokens, ahead, out):
        self.last_step = {"decodes": decodes, "prompt_tokens": prompt_tokens, "ahead": ahead}
        if self._log is not None:
            import json
            import time
            now = time.perf_counter()
            rec = dict(self.last_step, step=self.steps, produced=len(out), ms=round((now - self._log["t"]) * 1e3, 3),
                       running=len(self.scheduler.running), waiting=len(self.scheduler.waiting),
                       free_pages=self.runner.cache.free_pages())
            prof = getattr(self.runner.ops, "take_profile", None)
            if prof is not None:
                kernels = prof()
                if kernels:
                    rec["kernel_ms"] = kernels
            self._log["t"] = now
            self._log["f"].write(json.dumps(rec) + "\n")
            self._log["f"].flush()

    # ---- whole generation ------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[List[int]]:
        """Generated token ids for each prompt (token ids in, token ids out)."""
        if params is None or isinstance(params, SamplingParams):
            plist = [params or SamplingParams.greedy()] * len(prompts)
        else:
            plist = list(params)
        import copy
        ids = [self.add_request(p, copy.copy(sp)) for p, sp in zip(prompts, plist)]
        outs: Dict[int, List[int]] = {i: [] for i in ids}
        while self.scheduler.has_unfinished():
            res = self.step()
            if not res and not self.scheduler.has_unfinished():
                break
            for rid, tok, _ in res:
                if rid in outs:
                    outs[rid].append(tok)
        return [outs[i] for i in ids]

    def warm_up(self, max_batch: Optional[int] = None, max_context: Optional[int] = None, sampling: bool = False) -> int:
        """Capture every decode graph that requests up to these sizes can need (see
        ``ModelRunner.capture_decode_graphs``); serving then never stalls on a capture.
        ``sampling``: also the graphs that draw top-k / top-p tokens on the device."""
        return self.runner.capture_decode_graphs(max_batch, max_context, pool=sampling and self._device_pool)

    def stats(self) -> dict:
        s = self.scheduler.stats()
        s.update({"steps": self.steps, "generated": self.generated, "tokens_run": self.runner.tokens_run})
        return s


class Session:
    """One stream over the engine's model, after the reference's backend adapter
    (backend.rs:53-328): it owns its position; ``forward_logits`` feeds tokens in portions
    (backend.rs:185-232 cuts prompts into chunks of 512) and returns the last position's logits."""

    def __init__(self, runner: ModelRunner, chunk: Optional[int] = None):
        self.runner = runner
        self.chunk = min(chunk or 512, runner.max_rows)
        self.slot = runner.admit()
        if self.slot is None:
            raise RequestError("no free request slot for a session")

    @property
    def position(self) -> int:
        return self.runner.cached_len(self.slot)

    def forward_logits(self, tokens: Sequence[int]) -> torch.Tensor:
        tokens = list(tokens)
        if not tokens:
            raise RequestError("forward_logits needs at least one token")
        logits = None
        for i in range(0, len(tokens), self.chunk):
            piece = tokens[i:i + self.chunk]
            last = i + self.chunk >= len(tokens)
            logits = self.runner.step([StepEntry(self.slot, piece, (len(piece) - 1,) if last else ())])
        return logits[0].clone()

    def forward_all_logits(self, tokens: Sequence[int]) -> torch.Tensor:
        tokens = list(tokens)
        outs = []
        for i in range(0, len(tokens), self.chunk):
            piece = tokens[i:i + self.chunk]
            outs.append(self.runner.step([StepEntry(self.slot, piece, tuple(range(len(piece))))]).clone())
        return torch.cat(outs)

    def generate_token(self, tokens: Sequence[int]) -> int:
        lg = self.forward_logits(tokens)
        mx = lg.max()
        return int((lg == mx).nonzero()[0])

    def reset_position(self) -> None:
        self.runner.release(self.slot)
        self.slot = self.runner.admit()

    def truncate_to(self, n: int) -> None:
        """Keep the first ``n`` cached positions (backend.rs:95-114): the next call continues at n."""
        self.runner.truncate(self.slot, n)

    def close(self) -> None:
        if self.slot is not None:
            self.runner.release(self.slot)
            self.slot = None
