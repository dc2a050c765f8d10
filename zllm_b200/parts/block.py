"""Arrangements: the order in which a layer's norms, mixer and feed-forward act
on the residual stream.

``pre_norm`` is the Llama block: x <- x + mixer(norm1(x)); x <- x + ffn(norm2(x))
(zllm src/backend/candle/quantized_llama_fork.rs:943-958).  The residual stream
``x`` is float32; mixer and feed-forward add into it themselves so that a
product's epilogue can do the addition.
"""
from __future__ import annotations

from .base import register_arrangement


class Layer:
    """A built layer: its parts and its arrangement function."""

    def __init__(self, norm1, mixer, norm2, ffn, arrangement):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.arrangement = arrangement

    def parts(self):
        return {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "ffn": self.ffn}

    def run(self, x, ctx, cache, write_cache=True):
        self.arrangement(self, x, ctx, cache, write_cache)


@register_arrangement("pre_norm")
def pre_norm(layer: Layer, x, ctx, cache, write_cache):
    rt = layer.mixer.rt
    pro1 = layer.norm1.as_prologue() if layer.mixer.accepts_input_norm else None
    if pro1 is not None:
        layer.mixer.forward(x, x, ctx, cache, write_cache, input_norm=pro1)   # the norm runs inside the mixer's product
    else:
        h = ctx.ws.get("normed", tuple(x.shape), rt.dtype)
        layer.norm1.forward(x, h, ctx)
        layer.mixer.forward(h, x, ctx, cache, write_cache)
    pro2 = layer.norm2.as_prologue() if layer.ffn.accepts_input_norm else None
    if pro2 is not None:
        layer.ffn.forward(x, x, ctx, input_norm=pro2)
    else:
        h = ctx.ws.get("normed", tuple(x.shape), rt.dtype)
        layer.norm2.forward(x, h, ctx)
        layer.ffn.forward(h, x, ctx)
