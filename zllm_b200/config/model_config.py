"""Typed model configuration, read from the architecture's own ``config.json`` keys.

The reference reads hyper-parameters in one place and makes a missing mandatory
key a hard error that names the key (zllm src/backend/arch.rs:66-147; policy
stated at arch.rs:7-11).  Same here: no size and no constant that
``config.json`` gives has a stand-in in code; optional keys have exactly the
defaults the reference documents (kv heads = heads, head_dim = hidden / heads,
rope base 10000: arch.rs:120-146).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any, Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of the rotary encoding.

    ``llama3``: per-pair divisors computed from (factor, low_freq_factor,
    high_freq_factor, original_max_position_embeddings); the reference consumes
    such divisors from a tensor (fork.rs:584-590).  ``linear``: every frequency
    divided by ``factor`` (fork.rs:592-597).
    """

    rope_type: str
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0

    @staticmethod
    def from_dict(d: Optional[dict]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise ConfigError(f"config.json: rope_scaling must be an object or null, found {d!r}")
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind == "llama3":
            need = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
            for k in need:
                if k not in d:
                    raise ConfigError(f"config.json: rope_scaling (llama3) is missing key {k!r}")
            return RopeScaling("llama3", float(d["factor"]), float(d["low_freq_factor"]),
                               float(d["high_freq_factor"]), int(d["original_max_position_embeddings"]))
        if kind == "linear":
            if "factor" not in d:
                raise ConfigError("config.json: rope_scaling (linear) is missing key 'factor'")
            return RopeScaling("linear", float(d["factor"]))
        raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported (llama3, linear, default)")

    def to_dict(self) -> dict:
        if self.rope_type == "linear":
            return {"rope_type": "linear", "factor": self.factor}
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


_REQUIRED = (
    "num_hidden_layers",
    "hidden_size",
    "num_attention_heads",
    "intermediate_size",
    "vocab_size",
    "rms_norm_eps",
    "max_position_embeddings",
)


@dataclass(frozen=True)
class LlamaConfig:
    """The keys of a ``LlamaForCausalLM`` ``config.json``."""

    architecture: str
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Any = None
    extra: dict = field(default_factory=dict, compare=False)

    # ---- reading -------------------------------------------------------
    @staticmethod
    def from_dict(d: dict) -> "LlamaConfig":
        archs = d.get("architectures")
        if not archs or not isinstance(archs, list):
            raise ConfigError("config.json: missing key 'architectures' (a list with the model class name)")
        for k in _REQUIRED:
            if k not in d:
                raise ConfigError(f"config.json: missing mandatory key {k!r}")
        nh = _pos_int(d, "num_attention_heads")
        H = _pos_int(d, "hidden_size")
        nkv = int(d["num_key_value_heads"]) if d.get("num_key_value_heads") is not None else nh
        if d.get("head_dim") is not None:
            hd = int(d["head_dim"])
        else:
            if H % nh:
                raise ConfigError(f"config.json: hidden_size {H} is not divisible by num_attention_heads {nh} "
                                  "and no head_dim is given")
            hd = H // nh
        if nkv <= 0 or nh % nkv:
            raise ConfigError(f"config.json: num_attention_heads {nh} is not a multiple of num_key_value_heads {nkv}")
        if hd <= 0 or hd % 2:
            raise ConfigError(f"config.json: head_dim {hd} must be positive and even (rotary pairs)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (the Llama feed-forward is SiLU-gated)")
        for flag in ("attention_bias", "mlp_bias"):
            if d.get(flag, False):
                raise ConfigError(f"config.json: {flag}=true is not supported by LlamaForCausalLM here")
        eps = float(d["rms_norm_eps"])
        if not eps > 0:
            raise ConfigError(f"config.json: rms_norm_eps must be > 0, found {eps}")
        known = set(_REQUIRED) | {
            "architectures", "num_key_value_heads", "head_dim", "rope_theta", "rope_scaling",
            "tie_word_embeddings", "hidden_act", "attention_bias", "mlp_bias", "torch_dtype", "dtype",
            "bos_token_id", "eos_token_id",
        }
        extra = {k: v for k, v in d.items() if k not in known}
        return LlamaConfig(
            architecture=str(archs[0]),
            num_hidden_layers=_pos_int(d, "num_hidden_layers"),
            hidden_size=H,
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=hd,
            intermediate_size=_pos_int(d, "intermediate_size"),
            vocab_size=_pos_int(d, "vocab_size"),
            rms_norm_eps=eps,
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            max_position_embeddings=_pos_int(d, "max_position_embeddings"),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=act,
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=d.get("eos_token_id"),
            extra=extra,
        )

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d


def _pos_int(d: dict, key: str) -> int:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: key {key!r} must be a positive integer, found {v!r}")
    return v


def read_config_json(model_dir) -> dict:
    """The raw dictionary of ``<model_dir>/config.json``; ConfigError if unreadable."""
    path = Path(model_dir) / "config.json"
    try:
        text = path.read_text()
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    try:
        d = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d
