"""Engine settings: cache pool, batch limits, precision.

The reference splits these between its TOML file (``[memory] block_size = 16,
max_blocks``; zllm src/config.rs:71-75, configs/default.toml) and environment
flags (``ZLLM_CB_SLOTS`` = 16 slots, ``ZLLM_CB_SEQ``, ``ZLLM_PREFILL_CHUNK``;
src/main.rs:378-379, src/backend/candle/backend.rs:198-205).  Here they are one
typed record.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError

DTYPES = ("bfloat16", "float32")
MAX_SEQS = 1024                       # rows of one decode step (csrc/sampling.cu advance_decode_kernel)


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16": serving kernels; "float32": true 32-bit everywhere
    block_size: int = 16               # positions per cache page (reference DEFAULT_BLOCK_SIZE)
    num_blocks: Optional[int] = None   # pages per cache group; None: max_num_seqs full sequences
    max_num_seqs: int = 16             # live requests (slots); reference default ZLLM_CB_SLOTS=16
    max_num_batched_tokens: int = 2048  # token budget of one step
    max_model_len: Optional[int] = None  # None: the model's max_position_embeddings
    seed: int = 0
    device: str = "cuda:0"
    cuda_graphs: bool = True           # replay captured graphs for decode-only steps
    step_graphs: bool = True           # with cuda_graphs: also capture steps with prompt portions, per shape bucket
    prefix_sharing: bool = True        # requests take over the full cache pages of a prompt prefix seen before

    def validate(self) -> "EngineConfig":
        if self.dtype not in DTYPES:
            raise ConfigError(f"engine dtype {self.dtype!r} is not one of {DTYPES}")
        for k in ("block_size", "max_num_seqs", "max_num_batched_tokens"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"engine setting {k} must be a positive integer, found {v!r}")
        if self.max_num_seqs > MAX_SEQS:
            raise ConfigError(f"engine setting max_num_seqs is at most {MAX_SEQS} (one block of the decode-advance "
                              f"kernel covers a step's rows), found {self.max_num_seqs}")
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise ConfigError(f"engine setting num_blocks must be positive, found {self.num_blocks}")
        if self.max_model_len is not None and self.max_model_len <= 0:
            raise ConfigError(f"engine setting max_model_len must be positive, found {self.max_model_len}")
        return self
