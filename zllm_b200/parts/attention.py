"""Grouped-query attention over the paged cache.

q = Wq h, k = Wk h, v = Wv h without biases (zllm
src/backend/candle/quantized_llama_fork.rs:462-473); head ``i`` is columns
i*hd..(i+1)*hd-1 (fork.rs:475-487); q and k are rotated, v is not
(fork.rs:489-490); the new k and v go to the cache at their positions
(fork.rs:495-496) before any row attends; scores q.k / sqrt(hd), query head h
reads kv head h // (nh/nkv), key j visible to a query at position p iff j <= p
(and j > p - window when a window is set), softmax and the weighted sum in
float32 (fork.rs:518-533; src/backend/gpu/shaders.rs:703-723); heads concatenated
to [T, nh*hd], which may differ from the width (fork.rs:514-516); output
projection added to the residual (fork.rs:535,945).

The three projections are stacked into one matrix at load, as the reference's
Vulkan path concatenates weights to save a pass (src/backend/vulkan/mod.rs:1141-1181).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..errors import ConfigError
from .base import KVCacheSpec, Mixer, WeightSpec, register_mixer


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position_encoding=None, window: Optional[int] = None, scale: Optional[float] = None,
                 init_std: float = 0.02):
        if n_heads % n_kv_heads:
            raise ConfigError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if head_dim % 16:
            raise ConfigError(f"attention: head_dim {head_dim} must be a multiple of 16")
        self.hidden_size = int(hidden_size)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.position_encoding = position_encoding
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.init_std = init_std
        self.w_qkv = None
        self.w_o = None

    def weight_specs(self):
        H, hd = self.hidden_size, self.head_dim
        s = ("normal", self.init_std)
        return {
            "q_proj": WeightSpec((self.n_heads * hd, H), "matrix", s),
            "k_proj": WeightSpec((self.n_kv_heads * hd, H), "matrix", s),
            "v_proj": WeightSpec((self.n_kv_heads * hd, H), "matrix", s),
            "o_proj": WeightSpec((H, self.n_heads * hd), "matrix", s),
        }

    def cache_spec(self):
        return KVCacheSpec(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, rt):
        super().bind(rt)
        if self.position_encoding is not None and self.position_encoding.rt is None:
            self.position_encoding.bind(rt)

    def load(self, tensors):
        self.w_qkv = torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0).contiguous()
        self.w_o = tensors["o_proj"].contiguous()

    accepts_input_norm = True
    capturable = True

    def step_planner(self):
        # the tiled attention kernels want each portion cut into query tiles of their own size
        return getattr(self.rt.ops, "plan_query_tiles", None)

    def forward(self, h, residual, ctx, cache, write_cache: bool = True, input_norm=None):
        """``input_norm`` None: h is the normed input.  Otherwise h is the float32 residual and
        ``input_norm`` = (weight, eps) of the RMS norm to apply to it inside the QKV product."""
        ops = self.rt.ops
        T = h.shape[0]
        nq, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = ctx.ws.get("qkv", (T, (nq + 2 * nkv) * hd), self.rt.dtype)
        rot = self.position_encoding.rotary() if self.position_encoding is not None else None
        ops.qkv_rope_store(h, input_norm, self.w_qkv, qkv, ctx, rot, cache, nq, nkv, hd, write_cache, ctx.ws)
        att = ctx.ws.get("attn_out", (T, nq * hd), self.rt.dtype)
        ops.paged_attention(qkv, att, ctx, cache, nq, nkv, hd, self.scale, self.window)
        ops.linear(att, self.w_o, residual, "add")
