"""Per-request sampling settings and the per-token seed.

After zllm's two samplers: the batched path's ``SamplingParams{temp, top_k,
top_p}`` with ``greedy()`` / ``temperature(t)`` and a stateless per-token seed
``seed_n = base + n * 0x9E3779B1`` (src/backend/gpu/sampling.rs:7-21), and the
CLI's ``SamplerConfig`` which adds ``min_p`` (src/engine/sampler.rs:3-22).
``temperature <= 0`` means greedy in both (sampler.rs:35, sampling.rs:11).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

from ..errors import RequestError

TOPK_POOL = 64      # candidates the device extracts for top-k/top-p (reference TOPK_K, gpu/mod.rs:1846)
_M32 = 0xFFFFFFFF


@dataclass
class SamplingParams:
    temperature: float = 0.0        # <= 0: greedy (argmax, lowest index on ties)
    top_k: int = 0                  # 0: off
    top_p: float = 1.0              # >= 1 or 0: off
    min_p: float = 0.0              # 0: off; keep tokens with p >= min_p * p_max
    seed: int = 0
    max_tokens: int = 128
    stop_token_ids: Tuple[int, ...] = ()

    @staticmethod
    def greedy(max_tokens: int = 128, **kw) -> "SamplingParams":
        return SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw)

    @staticmethod
    def with_temperature(t: float, seed: int = 0, max_tokens: int = 128, **kw) -> "SamplingParams":
        return SamplingParams(temperature=t, seed=seed, max_tokens=max_tokens, **kw)

    def validate(self) -> "SamplingParams":
        if self.max_tokens < 1:
            raise RequestError(f"max_tokens must be at least 1, found {self.max_tokens}")
        if self.top_k < 0:
            raise RequestError(f"top_k must be >= 0, found {self.top_k}")
        if not (0.0 <= self.top_p):
            raise RequestError(f"top_p must be >= 0, found {self.top_p}")
        if not (0.0 <= self.min_p <= 1.0):
            raise RequestError(f"min_p must be in [0, 1], found {self.min_p}")
        self.stop_token_ids = tuple(int(t) for t in self.stop_token_ids)
        return self

    @property
    def is_greedy(self) -> bool:
        return not (self.temperature > 0.0)

    @property
    def needs_topk(self) -> bool:
        """The candidate-pool path (sampling.rs:21)."""
        return (not self.is_greedy) and (self.top_k > 0 or 0.0 < self.top_p < 1.0)

    @property
    def needs_full(self) -> bool:
        """Settings the 64-candidate pool cannot serve: min_p, or top_k beyond the pool."""
        return (not self.is_greedy) and (self.min_p > 0.0 or self.top_k > TOPK_POOL)


def step_seed(base: int, gen_index: int) -> int:
    """Seed of the ``gen_index``-th generated token (sampling.rs:9), 32-bit wrapping."""
    return (base + gen_index * 0x9E3779B1) & _M32
