"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees -- pure host logic over the cache manager.

States and rules follow the reference's ``ContinuousBatcher`` (zllm
src/backend/gpu/batch.rs):

* queues ``running`` (decoding), ``prefilling`` (FIFO), ``preempted`` (FIFO), free
  slots (batch.rs:48-62); here also ``waiting`` for requests that have no slot yet
  (the reference's server loop holds those in its channel, batch.rs:512-525).
* admission is optimistic: a free slot and room for the tokens to prefill
  (batch.rs:136-140,163-171); empty prompts and prompts beyond the maximum length
  are rejected (batch.rs:164).
* every running request contributes its last token (batch.rs:180-183); the first
  token of a request is produced by the step whose portion completes its prompt
  (batch.rs:327-334).
* a request finishes when it produces a stop token (which IS emitted) or reaches
  ``max_tokens`` (batch.rs:198-206); slot and pages are released in the same step.
* WHEN PAGES RUN OUT (batch.rs:262-310,323-326): before decoding, the most
  recently admitted running request is preempted (LIFO) until the rest can grow,
  never the last one; the FRONT prefilling request has priority -- running
  requests, then the newest other prefilling request, are preempted for its
  portion, and if that is not enough the portion is shortened to the pages there
  are, or waits.  A preempted request gives back all its pages and its slot and
  keeps its whole token history; it is resumed first-in-first-out when a slot is
  free and everything already admitted plus its own tokens fit, by prefilling
  prompt ++ produced tokens again (batch.rs:363-390).  Its sampling continues with
  the same generation index, hence the same seeds, hence the same tokens.

Beyond the reference: a per-step token budget ``max_num_batched_tokens``.  Decoded
tokens are scheduled first; what is left of the budget goes to prompt portions,
of several requests if it reaches, and everything runs in ONE forward.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..errors import MemoryError_, RequestError
from ..sampling.params import SamplingParams, step_seed

WAITING, PREFILLING, RUNNING, PREEMPTED, FINISHED = "waiting", "prefilling", "running", "preempted", "finished"


@dataclass
class Request:
    id: int
    tokens: List[int]                 # prompt ++ every produced token
    prompt_len: int
    params: SamplingParams
    slot: Optional[int] = None
    num_computed: int = 0             # positions of ``tokens`` that are in the cache
    state: str = WAITING
    finish_reason: Optional[str] = None

    @property
    def gen_index(self) -> int:
        return len(self.tokens) - self.prompt_len

    def next_seed(self) -> int:
        return step_seed(self.params.seed, self.gen_index)


@dataclass
class Portion:
    request: Request
    start: int
    n: int
    completes: bool                   # the portion reaches the end of the tokens to prefill


@dataclass
class Plan:
    decodes: List[Request] = field(default_factory=list)
    portions: List[Portion] = field(default_factory=list)

    @property
    def empty(self) -> bool:
        return not self.decodes and not self.portions

    @property
    def num_tokens(self) -> int:
        return len(self.decodes) + sum(p.n for p in self.portions)


class Scheduler:
    def __init__(self, cache, max_num_batched_tokens: int, max_model_len: int):
        self.cache = cache
        self.budget = int(max_num_batched_tokens)
        self.max_len = int(max_model_len)
        self.waiting: Deque[Request] = deque()
        self.prefilling: Deque[Request] = deque()
        self.running: List[Request] = []          # in order of admission
        self.preempted: Deque[Request] = deque()
        self.requests: Dict[int, Request] = {}
        self.preemptions = 0
        self.finished = 0
        self._next_id = 0

    # ---- requests ------------------------------------------------------
    def add(self, prompt: Sequence[int], params: SamplingParams, request_id: Optional[int] = None) -> int:
        params.validate()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise RequestError("empty prompt")
        if len(prompt) >= self.max_len:
            raise RequestError(f"prompt of {len(prompt)} tokens leaves no room under the maximum length {self.max_len}")
        worst = min(len(prompt) + params.max_tokens, self.max_len)
        total = [g.pool.num_pages for g in self.cache.groups]
        if any(n > t for n, t in zip(self.cache.pages_short(None, worst), total)):
            raise RequestError(f"request of up to {worst} positions can never fit the cache pool ({total} pages)")
        if request_id is None:
            request_id = self._next_id
        if request_id in self.requests:
            raise RequestError(f"request id {request_id} is in use")
        self._next_id = max(self._next_id, request_id + 1)
        r = Request(request_id, prompt, len(prompt), params)
        self.requests[request_id] = r
        self.waiting.append(r)
        return request_id

    def cancel(self, request_id: int) -> bool:
        """Remove a request wherever it is; its slot and pages are free at once (batch.rs:87-105)."""
        r = self.requests.get(request_id)
        if r is None or r.state == FINISHED:
            return False
        for q in (self.waiting, self.prefilling, self.preempted):
            if r in q:
                q.remove(r)
        if r in self.running:
            self.running.remove(r)
        self._finish(r, "cancelled")
        return True

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.prefilling or self.running or self.preempted)

    # ---- planning ---------------------------------------------------------
    def _demand(self, r: Request, upto: Optional[int] = None) -> Tuple[Optional[int], int]:
        return (r.slot, len(r.tokens) if upto is None else upto)

    def _admit(self) -> None:
        """Resume preempted requests, then admit waiting ones, first in first out, while a slot
        is free and what is admitted already plus the newcomer's tokens fit."""
        for queue in (self.preempted, self.waiting):
            while queue and self.cache.has_free_slot():
                r = queue[0]
                held = [self._demand(x) for x in self.running] + [self._demand(x) for x in self.prefilling]
                if not self.cache.can_fit(held + [(None, len(r.tokens))]):
                    return                      # keep the order: nobody overtakes the head
                queue.popleft()
                r.slot = self.cache.admit()
                # full pages of a prefix that an earlier request left registered are taken over
                r.num_computed = self.cache.adopt_prefix(r.slot, r.tokens)
                r.state = PREFILLING
                self.prefilling.append(r)

    def _preempt(self, r: Request) -> None:
        self.cache.free_slot(r.slot)
        r.slot = None
        r.num_computed = 0
        r.state = PREEMPTED
        self.preempted.append(r)
        self.preemptions += 1

    def _preempt_last_running(self) -> bool:
        if not self.running:
            return False
        self._preempt(self.running.pop())
        return True

    def _preempt_last_prefilling(self) -> bool:
        if len(self.prefilling) < 2:
            return False
        self._preempt(self.prefilling.pop())
        return True

    def schedule(self) -> Plan:
        self._admit()
        plan = Plan()
        # decoded tokens first: every running request grows by one position
        while len(self.running) > 1 and not self.cache.can_fit([self._demand(r) for r in self.running]):
            self._preempt_last_running()
        if len(self.running) == 1 and not self.cache.can_fit([self._demand(self.running[0])]):
            while self.prefilling and not self.cache.can_fit([self._demand(self.running[0])]):
                self._preempt(self.prefilling.pop())
            if not self.cache.can_fit([self._demand(self.running[0])]):
                raise MemoryError_("the cache pool cannot hold the single running request")
        while len(self.running) > self.budget:
            self._preempt_last_running()
        plan.decodes = list(self.running)
        left = self.budget - len(plan.decodes)
        # prompt portions with what is left of the budget
        demands = [self._demand(r) for r in plan.decodes]
        i = 0
        while i < len(self.prefilling) and left > 0:
            r = self.prefilling[i]
            n = min(len(r.tokens) - r.num_computed, left)
            front = i == 0
            while n > 0 and not self.cache.can_fit(demands + [self._demand(r, r.num_computed + n)]):
                if front and plan.decodes and self._preempt_last_running():
                    plan.decodes.pop()
                    demands = [self._demand(x) for x in plan.decodes] + \
                              [self._demand(p.request, p.start + p.n) for p in plan.portions]
                    left += 1
                    n = min(len(r.tokens) - r.num_computed, left)
                elif front and self._preempt_last_prefilling():
                    pass
                else:
                    n = self._largest_fit(r, n, demands)
                    break
            if n <= 0:
                break                            # wait: pages come back when others finish
            plan.portions.append(Portion(r, r.num_computed, n, r.num_computed + n == len(r.tokens)))
            demands.append(self._demand(r, r.num_computed + n))
            left -= n
            i += 1
        return plan

    def _largest_fit(self, r: Request, n: int, demands) -> int:
        lo, hi = 0, n                            # can_fit is monotone in the portion's length
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.cache.can_fit(demands + [self._demand(r, r.num_computed + mid)]):
                lo = mid
            else:
                hi = mid - 1
        return lo

    # ---- after the forward ---------------------------------------------------
    def commit(self, plan: Plan, decode_tokens: Sequence[int], first_tokens: Sequence[Optional[int]]):
        """Record the step's results.  ``decode_tokens[i]`` belongs to ``plan.decodes[i]``;
        ``first_tokens[j]`` to ``plan.portions[j]`` (None unless the portion completes).
        Returns [(request id, token, done)] in that order."""
        out = []
        for r, tok in zip(plan.decodes, decode_tokens):
            r.num_computed += 1
            self.cache.register_prefix(r.slot, r.tokens, r.num_computed)
            out.append(self._produce(r, int(tok)))
        for p, tok in zip(plan.portions, first_tokens):
            r = p.request
            r.num_computed += p.n
            self.cache.register_prefix(r.slot, r.tokens, r.num_computed)
            if p.completes:
                self.prefilling.remove(r)
                r.state = RUNNING
                self.running.append(r)
                out.append(self._produce(r, int(tok)))
        return out

    def _produce(self, r: Request, tok: int):
        r.tokens.append(tok)
        reason = None
        if tok in r.params.stop_token_ids:
            reason = "stop"
        elif r.gen_index >= r.params.max_tokens:
            reason = "length"
        elif len(r.tokens) >= self.max_len:
            reason = "max_model_len"
        if reason:
            self.running.remove(r)
            self._finish(r, reason)
        return (r.id, tok, reason is not None)

    def _finish(self, r: Request, reason: str) -> None:
        if r.slot is not None:
            self.cache.free_slot(r.slot)
            r.slot = None
        r.state = FINISHED
        r.finish_reason = reason
        self.finished += 1

    def stats(self) -> dict:
        return {"waiting": len(self.waiting), "prefilling": len(self.prefilling), "running": len(self.running),
                "preempted": len(self.preempted), "preemptions": self.preemptions, "finished": self.finished,
                "free_pages": self.cache.free_pages(), "free_slots": len(self.cache.free_slots),
                "prefix_hits": self.cache.prefix_hits, "prefix_misses": self.cache.prefix_misses}
