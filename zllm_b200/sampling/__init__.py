from .params import SamplingParams, TOPK_POOL, step_seed
from .sampler import Sampler, rng01, sample_from_pool, sample_full

__all__ = ["SamplingParams", "TOPK_POOL", "step_seed", "Sampler", "rng01", "sample_from_pool", "sample_full"]
