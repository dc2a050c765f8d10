"""Random-weights mode: a model folder from a configuration and a seed.

The reference has no such mode (its tests need a real model file or a fake
backend, zllm src/backend/dummy.rs:67-73); benchmarks and tests here need
models of any size without a download.  Every tensor is drawn on the CPU from a
generator seeded by (seed, tensor name), so a tensor's values do not depend on
which other tensors exist or in which order they are drawn.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from ..parts.base import WeightSpec
from .safetensors_io import write_safetensors

_STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: WeightSpec, seed: int, dtype=torch.float32, device="cpu",
                  std: float | None = None, norm_std: float | None = None) -> torch.Tensor:
    kind, own_std = spec.init
    if kind == "one_plus_normal":
        std = norm_std if norm_std is not None else own_std
    elif std is None:
        std = own_std
    if str(device) == "cpu":
        g = torch.Generator(device="cpu").manual_seed(_tensor_seed(seed, name))
        t = torch.randn(spec.shape, generator=g, dtype=torch.float32)
    else:
        g = torch.Generator(device=device).manual_seed(_tensor_seed(seed, name))
        t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    t = t * std
    if kind == "one_plus_normal":
        t = t + 1.0
    return t.to(dtype)


def random_state(expected: Mapping[str, WeightSpec], seed: int, dtype=torch.float32, device="cpu",
                 std: float | None = None, norm_std: float | None = None) -> Dict[str, torch.Tensor]:
    return {n: random_tensor(n, s, seed, dtype, device, std, norm_std) for n, s in expected.items()}


def write_random_model(model_dir, config, seed: int, dtype: str = "float32", std: float | None = None,
                       norm_std: float = 0.0) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a typed configuration.

    ``std`` overrides the matrices' standard deviation (default 0.02); norm weights
    are 1 + N(0, norm_std).  Values are drawn in float32 and stored as ``dtype``.
    """
    from ..config.registry import architecture
    from ..models.decoder import expected_tensors

    spec = architecture(config.architecture).build_spec(config)
    expected = expected_tensors(spec)
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = dtype
    (model_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    tensors = random_state(expected, seed, _STORE[dtype], "cpu", std, norm_std)
    write_safetensors(model_dir / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return model_dir
