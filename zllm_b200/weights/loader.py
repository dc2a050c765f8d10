"""Weights by tensor name, checked against what the model expects.

The reference names a tensor in every load failure (zllm
src/backend/gpu/mod.rs:1402, src/backend/candle/backend.rs:343-365) and treats a
missing output matrix as "tied to the embedding" (quantized_llama_fork.rs:761-764).
Here all problems of a folder are collected and raised as ONE error that lists
missing tensors, unexpected tensors and wrong shapes.

Dtypes: a tensor stays as stored -- bfloat16 stays bfloat16, a tensor stored in
32-bit stays 32-bit, integer tables become int32 -- with two exceptions that
the roles of ``WeightSpec`` state: in the float32 engine every floating tensor
is widened to float32 (exact), and in the bfloat16 engine a *matrix* or
*embedding* stored wider than bfloat16 is rounded to it, because the
tensor-core products take bfloat16 operands.
"""
from __future__ import annotations

from fnmatch import fnmatchcase
from typing import Dict, Mapping, Tuple

import torch

from ..errors import ModelError
from ..parts.base import WeightSpec
from .safetensors_io import open_model_files


def target_dtype(stored: torch.dtype, role: str, engine_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if role in ("matrix", "embedding"):
        return engine_dtype
    # vectors and other small tensors: as stored; half precision has no kernels, widen it
    return torch.float32 if stored in (torch.float16, torch.float64) else stored


def check_names(expected: Mapping[str, WeightSpec], found: Mapping[str, Tuple[torch.dtype, Tuple[int, ...]]],
                optional: Mapping[str, WeightSpec] = None, ignored=()) -> None:
    """Raise one ModelError listing every missing, unexpected and mis-shaped tensor.

    ``optional``: tensors that may be absent (checked like the others when present).
    ``ignored``: fnmatch patterns of names a folder may hold and nobody reads."""
    optional = optional or {}
    missing = [n for n in expected if n not in found]
    unexpected = [n for n in found if n not in expected and n not in optional
                  and not any(fnmatchcase(n, pat) for pat in ignored)]
    wrong = []
    for n, spec in list(expected.items()) + list(optional.items()):
        if n in found and tuple(found[n][1]) != tuple(spec.shape):
            wrong.append(f"{n}: expected {list(spec.shape)}, found {list(found[n][1])}")
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append(f"missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            parts.append(f"wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise ModelError("model weights do not match the configuration -- " + " | ".join(parts))


def load_checked(model_dir, expected: Mapping[str, WeightSpec], engine_dtype: torch.dtype, device,
                 optional: Mapping[str, WeightSpec] = None, ignored=()) -> Dict[str, torch.Tensor]:
    """Read every expected tensor, and every optional one that is there, from the folder onto
    ``device`` in its target dtype."""
    where = open_model_files(model_dir)
    try:
        found = {n: f.meta(n) for n, f in where.items()}
        check_names(expected, found, optional, ignored)
        out = {}
        for name, spec in list(expected.items()) + list((optional or {}).items()):
            if name not in where:
                continue
            t = where[name].tensor(name)
            out[name] = t.to(device=device, dtype=target_dtype(t.dtype, spec.role, engine_dtype)).contiguous()
    finally:
        for f in {id(f): f for f in where.values()}.values():
            f.close()           # tensors that are still views keep the file's map alive themselves
    return out
