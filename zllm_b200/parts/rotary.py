"""Rotary position encoding: tables of cos/sin(pos * theta_j) and the pairing.

theta_j = base^(-2j/rot_dim), optionally divided by per-pair divisors
(zllm src/backend/candle/quantized_llama_fork.rs:579-590); tables for positions
0..max_position as the float32 product pos * theta_j followed by cos/sin
(fork.rs:631-638).  The reference receives llama3 divisors precomputed in the
model file; from ``rope_scaling`` of a config.json they are computed here: with
wavelength lambda_j = 2 pi / theta_j, f_j = 1 below L/high, F above L/low, and a
linear blend of theta_j/F and theta_j in between.  ``linear`` scaling divides
every theta_j by the factor (fork.rs:592-597).

Pairing: ``interleaved`` rotates (x[2j], x[2j+1]) (the reference's ``rope_i``,
shaders.rs:576-586); otherwise (x[j], x[j + rot_dim/2]) (its ``rope_neox``,
fork.rs:447-451), which is the layout of unpermuted safetensors weights.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from ..errors import ConfigError
from .base import PositionEncoding, register_position_encoding


@dataclass
class RotaryTables:
    cos: torch.Tensor          # [max_position, rot_dim/2] float32, on device
    sin: torch.Tensor
    rot_dim: int
    interleaved: bool
    max_position: int


def inverse_frequencies(rot_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """theta_j in float64 (rounded to float32 by the caller)."""
    j = torch.arange(0, rot_dim, 2, dtype=torch.float64)
    inv = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -j / rot_dim)
    if not scaling:
        return inv
    kind = scaling.get("rope_type")
    if kind == "linear":
        return inv / float(scaling["factor"])
    if kind == "llama3":
        F = float(scaling["factor"])
        lo = float(scaling["low_freq_factor"])
        hi = float(scaling["high_freq_factor"])
        L = float(scaling["original_max_position_embeddings"])
        if hi <= lo:
            raise ConfigError("rope_scaling (llama3): high_freq_factor must exceed low_freq_factor")
        wavelen = 2.0 * math.pi / inv
        smooth = (L / wavelen - lo) / (hi - lo)
        blended = (1.0 - smooth) * inv / F + smooth * inv
        out = torch.where(wavelen < L / hi, inv, torch.where(wavelen > L / lo, inv / F, blended))
        return out
    raise ConfigError(f"rotary scaling {kind!r} is not supported (llama3, linear)")


@register_position_encoding("rotary")
class Rotary(PositionEncoding):
    def __init__(self, rot_dim: int, theta: float, max_position: int, scaling: Optional[dict] = None,
                 interleaved: bool = False, freq_factors=None):
        if rot_dim <= 0 or rot_dim % 2:
            raise ConfigError(f"rotary: rot_dim {rot_dim} must be positive and even")
        self.rot_dim = int(rot_dim)
        self.theta = float(theta)
        self.max_position = int(max_position)
        self.scaling = scaling
        self.interleaved = bool(interleaved)
        inv = inverse_frequencies(self.rot_dim, self.theta, scaling)
        if freq_factors is not None:
            # explicit divisors, the reference's own mechanism (fork.rs:584-590); 0 means "leave"
            ff = torch.as_tensor(freq_factors, dtype=torch.float64)
            if ff.numel() != inv.numel():
                raise ConfigError(f"rotary: {ff.numel()} freq_factors for {inv.numel()} pairs")
            inv = torch.where(ff != 0, inv / torch.where(ff != 0, ff, torch.ones_like(ff)), inv)
        self.inv_freq = inv.to(torch.float32)
        self._tables = None

    def bind(self, rt):
        super().bind(rt)
        pos = torch.arange(self.max_position, dtype=torch.float32)
        ang = pos[:, None] * self.inv_freq[None, :]          # float32 product, as the reference
        self._tables = RotaryTables(ang.cos().contiguous().to(rt.device), ang.sin().contiguous().to(rt.device),
                                    self.rot_dim, self.interleaved, self.max_position)

    def rotary(self):
        return self._tables
