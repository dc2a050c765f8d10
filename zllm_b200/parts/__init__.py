from .base import (FeedForward, KVCacheSpec, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec,
                   PositionEncoding, RunEntry, StateSpec, WeightSpec, build_part, register_arrangement,
                   register_feed_forward, register_mixer, register_norm, register_position_encoding,
                   registered)
from . import norm, rotary, attention, feedforward, block  # noqa: F401  (register the built-in kinds)
from .block import Layer

__all__ = ["FeedForward", "KVCacheSpec", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec",
           "PositionEncoding", "RunEntry", "StateSpec", "WeightSpec", "build_part", "register_arrangement",
           "register_feed_forward", "register_mixer", "register_norm", "register_position_encoding",
           "registered", "Layer"]
