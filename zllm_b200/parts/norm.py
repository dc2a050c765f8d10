"""RMSNorm.

y = x * rsqrt(mean_i(x_i^2) + eps) * w, the mean over the row, eps inside the
root, the weight applied after normalisation, no bias and no ``1 + w``
(zllm src/backend/gpu/shaders.rs:555-562; placement before attention, before the
feed-forward and before the head: quantized_llama_fork.rs:943,956,971).  Input is
the float32 residual stream; sums and the root are float32 in every path.
"""
from __future__ import annotations

from .base import Norm, WeightSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    capturable = True

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.size,), "vector", ("one_plus_normal", 0.0))}

    def forward(self, x, out, ctx):
        self.rt.ops.rmsnorm(x, self.weight, self.eps, out)
        return out

    def as_prologue(self):
        """(weight, eps): what a product needs to apply this norm to its own input rows."""
        return (self.weight, self.eps)
