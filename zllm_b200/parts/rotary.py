"""Rotary position encoding: tables of cos/sin(pos * theta_j) and the pairing.

theta_j = base^(-2j/rot_dim), optionally divided by per-pair divisors, all in
float32 (zllm src/backend/candle/quantized_llama_fork.rs:579-590); tables for
positions 0..max_position as the float32 product pos * theta_j followed by
cos/sin (fork.rs:631-638).  The reference receives llama3 divisors precomputed in the
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


def frequency_divisors(rot_dim: int, theta: float, scaling: Optional[dict]) -> Optional[torch.Tensor]:
    """The per-pair divisors f_j of ``llama3`` scaling, float32, as a model file would store them
    (the reference reads them from ``rope_freqs.weight``, fork.rs:584-590, 722-734); None when the
    scaling has none.  This is the converter's share of the work, so it is done in double precision
    and rounded once: f_j = 1 where the wavelength is below L/high, F above L/low, and in between
    theta_j / ((1 - s) theta_j / F + s theta_j) with s = (L / wavelength - low) / (high - low)."""
    if not scaling or scaling.get("rope_type") != "llama3":
        return None
    F = float(scaling["factor"])
    lo = float(scaling["low_freq_factor"])
    hi = float(scaling["high_freq_factor"])
    L = float(scaling["original_max_position_embeddings"])
    if hi <= lo:
        raise ConfigError("rope_scaling (llama3): high_freq_factor must exceed low_freq_factor")
    j = torch.arange(0, rot_dim, 2, dtype=torch.float64)
    wavelen = 2.0 * math.pi * torch.pow(torch.tensor(float(theta), dtype=torch.float64), j / rot_dim)
    smooth = (L / wavelen - lo) / (hi - lo)
    blend = 1.0 / ((1.0 - smooth) / F + smooth)
    one = torch.ones_like(wavelen)
    return torch.where(wavelen < L / hi, one, torch.where(wavelen > L / lo, one * F, blend)).to(torch.float32)


def inverse_frequencies(rot_dim: int, theta: float, scaling: Optional[dict], freq_factors=None) -> torch.Tensor:
    """theta_j in float32, computed as the reference computes it: 1 / base^(i / rot_dim) with
    every operand float32 (fork.rs:579-583), then divided by the divisors that are not zero
    (fork.rs:584-590), then ``linear`` scaling as a multiplication by 1 / factor (fork.rs:592-597)."""
    f32 = torch.float32
    i = torch.arange(0, rot_dim, 2, dtype=f32)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=f32), i / torch.tensor(float(rot_dim), dtype=f32))
    kind = scaling.get("rope_type") if scaling else None
    if kind not in (None, "default", "llama3", "linear"):
        raise ConfigError(f"rotary scaling {kind!r} is not supported (llama3, linear)")
    for div in (frequency_divisors(rot_dim, theta, scaling),
                torch.as_tensor(freq_factors, dtype=f32) if freq_factors is not None else None):
        if div is None:
            continue
        if div.numel() != inv.numel():
            raise ConfigError(f"rotary: {div.numel()} frequency divisors for {inv.numel()} pairs")
        inv = torch.where(div != 0, inv / torch.where(div != 0, div, torch.ones_like(div)), inv)
    if kind == "linear":
        inv = inv * (torch.tensor(1.0, dtype=f32) / max(float(scaling["factor"]), 1e-6))
    return inv


@register_position_encoding("rotary")
class Rotary(PositionEncoding):
    capturable = True

    def __init__(self, rot_dim: int, theta: float, max_position: int, scaling: Optional[dict] = None,
                 interleaved: bool = False, freq_factors=None):
        if rot_dim <= 0 or rot_dim % 2:
            raise ConfigError(f"rotary: rot_dim {rot_dim} must be positive and even")
        self.rot_dim = int(rot_dim)
        self.theta = float(theta)
        self.max_position = int(max_position)
        self.scaling = scaling
        self.interleaved = bool(interleaved)
        # explicit divisors are the reference's own mechanism (fork.rs:584-590); 0 means "leave"
        self.inv_freq = inverse_frequencies(self.rot_dim, self.theta, scaling, freq_factors)
        self._tables = None

    def bind(self, rt):
        super().bind(rt)
        pos = torch.arange(self.max_position, dtype=torch.float32)
        ang = pos[:, None] * self.inv_freq[None, :]          # float32 product, as the reference
        self._tables = RotaryTables(ang.cos().contiguous().to(rt.device), ang.sin().contiguous().to(rt.device),
                                    self.rot_dim, self.interleaved, self.max_position)

    def rotary(self):
        return self._tables
