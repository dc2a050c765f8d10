"""SiLU-gated feed-forward (SwiGLU), dense.

x <- x + Wdown( silu(Wgate h) * (Wup h) ), silu(g) = g / (1 + exp(-g)), no
biases (zllm src/backend/candle/quantized_llama_fork.rs:394-400,956-958;
src/backend/gpu/shaders.rs:984-988).  Gate and up are stored as one matrix so a
single product serves both, as the reference's Vulkan path does
(src/backend/vulkan/mod.rs:1141-1167); rows are interleaved in groups of eight
(eight gate rows, then the eight up rows of the same outputs) so that the
product's epilogue holds a gate value and its up value in the same thread and
writes silu(gate)*up directly.  An intermediate size that is no multiple of
eight keeps the two matrices apart and uses the stand-alone SiLU-mul kernel.
"""
from __future__ import annotations

import torch

from .base import FeedForward, WeightSpec, register_feed_forward

GATE_UP_GROUP = 8


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int = GATE_UP_GROUP) -> torch.Tensor:
    """[I,K],[I,K] -> [2I,K]: rows g*2*group .. : ``group`` gate rows then their ``group`` up rows."""
    I, K = gate.shape
    assert I % group == 0
    g = gate.reshape(I // group, group, K)
    u = up.reshape(I // group, group, K)
    return torch.stack([g, u], dim=1).reshape(2 * I, K).contiguous()


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, init_std: float = 0.02):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.init_std = init_std
        self.fused = self.intermediate_size % GATE_UP_GROUP == 0
        self.w_gate_up = None
        self.w_gate = None
        self.w_up = None
        self.w_down = None

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        s = ("normal", self.init_std)
        return {
            "gate_proj": WeightSpec((I, H), "matrix", s),
            "up_proj": WeightSpec((I, H), "matrix", s),
            "down_proj": WeightSpec((H, I), "matrix", s),
        }

    def load(self, tensors):
        if self.fused:
            self.w_gate_up = interleave_gate_up(tensors["gate_proj"], tensors["up_proj"])
        else:
            self.w_gate = tensors["gate_proj"].contiguous()
            self.w_up = tensors["up_proj"].contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    accepts_input_norm = True
    capturable = True

    def forward(self, h, residual, ctx, input_norm=None):
        """``input_norm`` as for the attention mixer: (weight, eps) when h is the float32 residual."""
        ops = self.rt.ops
        T = h.shape[0]
        act = ctx.ws.get("ffn_act", (T, self.intermediate_size), self.rt.dtype)
        if self.fused and input_norm is not None:
            ops.linear_normed(h, input_norm[0], input_norm[1], self.w_gate_up, act, "swiglu", ctx.ws)
        elif self.fused:
            ops.linear(h, self.w_gate_up, act, "swiglu")
        else:
            if input_norm is not None:
                hn = ctx.ws.get("normed", tuple(h.shape), self.rt.dtype)
                ops.rmsnorm(h, input_norm[0], input_norm[1], hn)
                h = hn
            up = ctx.ws.get("ffn_up", (T, self.intermediate_size), self.rt.dtype)
            ops.linear(h, self.w_gate, act, "store")
            ops.linear(h, self.w_up, up, "store")
            ops.silu_mul(act, up, act)
        ops.linear(act, self.w_down, residual, "add")
