"""What a part is: the interfaces of mixers, feed-forwards, norms, position
encodings and block arrangements, their registries, and the specs a model is
listed with.

The reference parameterises one forward by flags on an ``ArchSpec`` instead of
forking it per family (zllm src/backend/arch.rs:16-35).  This goes one step
further: a model is *data* -- a list of layers, each naming its mixer, its
feed-forward, its norms and their arrangement by registered kind, each kind
taking all its sizes and constants as parameters -- plus a run order that may
name a layer twice or let an entry read another entry's cache.  No part knows
which model it sits in; a part sees only its parameters, its own tensors, the
step's batch description and the cache view it was given.

Interfaces (all tensors are torch tensors on the engine's device):

``Norm.forward(x, out, ctx)``
    x [T, H] float32 residual stream -> out [T, H] in the compute dtype.
``Mixer.forward(h, residual, ctx, cache)``
    h [T, H] compute dtype (already normed); adds its result into ``residual``
    [T, H] float32 (the residual sum stays 32-bit).  ``cache`` is what the cache
    manager made from ``cache_spec()``: a ``KVLayerView``, a ``StateView`` or None.
``FeedForward.forward(h, residual, ctx)``
    same contract without a cache.
``PositionEncoding``
    hands the mixer what it needs to encode positions (for rotary encodings
    the cos/sin tables and pairing) and may act on the embedding output.
``Block`` arrangement
    given norms, mixer and feed-forward, runs them in its order on the residual.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..errors import ConfigError

# --------------------------------------------------------------------------
# specs (pure data)
# --------------------------------------------------------------------------


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part owns.

    role: "matrix" / "embedding" follow the engine's compute dtype (bfloat16 in
    serving, float32 in the 32-bit path); "vector" keeps the stored dtype
    (a tensor stored in 32-bit stays so) and is only widened in the 32-bit path;
    "int" tables become int32.
    init: ("normal", std) or ("one_plus_normal", std) for the random-weights mode.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple[str, float] = ("normal", 0.02)


@dataclass
class PartSpec:
    """A registered kind with its parameters, e.g. PartSpec("rmsnorm", {"size": 64, "eps": 1e-5})."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One layer: which parts it is made of and how they are arranged.

    ``tensor_names`` maps "<part>.<local tensor name>" (part in mixer, ffn,
    norm1, norm2) to the tensor's name in the model folder.
    """

    mixer: PartSpec
    ffn: PartSpec
    norm1: PartSpec
    norm2: PartSpec
    arrangement: str = "pre_norm"
    tensor_names: Dict[str, str] = field(default_factory=dict)


@dataclass
class RunEntry:
    """One entry of the run order.  ``layer`` indexes ``ModelSpec.layers``;
    ``cache_of`` is None when the entry owns its cache, else the index of the
    earlier run entry whose cache it reads (it then writes none)."""

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    """A whole decoder as data."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_position: int
    layers: List[LayerSpec]
    run_order: List[RunEntry]
    final_norm: PartSpec
    embedding_name: str
    final_norm_names: Dict[str, str]
    head_name: Optional[str]            # None: the head is always the embedding table
    init_std: float = 0.02
    norm_init_std: float = 0.0          # norm weights 1 + N(0, this) in random mode
    # a position encoding that acts on the embedding output (absolute encodings); encodings that
    # act inside a mixer (rotary) are parameters of that mixer instead
    embedding_position: Optional[PartSpec] = None
    embedding_position_names: Dict[str, str] = field(default_factory=dict)
    # True: a folder may lack ``head_name``, and the head is then the embedding table.  The tensor's
    # presence decides, as in the reference (quantized_llama_fork.rs:761-764), not a flag.
    head_optional: bool = False
    # what the configuration says about tying: the random-weights mode writes no head tensor when
    # true; at load a disagreement with what the folder holds is warned about, presence wins
    tie_head: bool = False
    # fnmatch patterns of tensors a folder may hold and the model does not read
    ignored_tensors: Tuple[str, ...] = ()
    # token ids that end a generation unless the caller says otherwise (a model's end-of-text ids)
    stop_token_ids: Tuple[int, ...] = ()


# --------------------------------------------------------------------------
# cache needs a mixer can declare
# --------------------------------------------------------------------------


@dataclass(frozen=True)
class KVCacheSpec:
    """Keys and values of every position (window None) or of the last ``window``."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one array of ``shape`` per request slot."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


# --------------------------------------------------------------------------
# part base classes
# --------------------------------------------------------------------------


class Part:
    """Base of all parts.  ``rt`` (set by ``bind``) gives dtype, device and kernels."""

    rt = None

    # True: ``forward`` only launches work on the current stream and learns about the step from
    # ``ctx``'s device arrays and shapes alone (never from ``ctx.entries`` or other host data), so
    # a step with prompt portions may be captured as a CUDA graph and replayed for other steps of
    # the same shape.  Decode-only steps are captured whatever this says (there ``ctx.entries`` is
    # None and a part must already manage with the device arrays).
    capturable = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def bind(self, rt) -> None:
        self.rt = rt

    def load(self, tensors: Dict[str, Any]) -> None:
        """Receive own tensors (local names), already on device in the dtype their role asks."""
        for k, v in tensors.items():
            setattr(self, k, v)

    def step_planner(self):
        """None, or a callable ``(entries, starts, aux) -> {name: (offset, shape)}`` that is run on
        the host once per step outside captured graphs: it writes integer tables its kernels want
        (cut from ``aux.take(n)``, a piece of the step's one upload) and names them; the forward
        finds them as ``ctx.aux[name]`` on the device.  Parts that return equal callables share one
        run.  Steps replayed from a graph (single decoded tokens only) run no planner."""
        return None


class Norm(Part):
    def forward(self, x, out, ctx):
        raise NotImplementedError

    def as_prologue(self):
        """(weight, eps) if a following product may apply this norm itself (an RMS norm), else None."""
        return None


class PositionEncoding(Part):
    def rotary(self):
        """A ``RotaryTables`` for mixers that rotate queries and keys, or None."""
        return None

    def on_embedding(self, x, ctx):
        """Act on the embedding output (absolute encodings); default nothing."""
        return None


class Mixer(Part):
    # True: ``forward`` takes ``input_norm=(weight, eps)`` and then receives the float32 residual
    # itself as ``h`` (it applies the norm inside its first product)
    accepts_input_norm = False

    def cache_spec(self):
        return None

    def forward(self, h, residual, ctx, cache, write_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    accepts_input_norm = False          # as for Mixer

    def forward(self, h, residual, ctx):
        raise NotImplementedError


# --------------------------------------------------------------------------
# registries
# --------------------------------------------------------------------------

_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "arrangement": {},
}


def _register(group: str, kind: str):
    def deco(obj):
        _REGISTRIES[group][kind] = obj
        return obj
    return deco


def register_mixer(kind): return _register("mixer", kind)
def register_feed_forward(kind): return _register("feed_forward", kind)
def register_norm(kind): return _register("norm", kind)
def register_position_encoding(kind): return _register("position_encoding", kind)
def register_arrangement(kind): return _register("arrangement", kind)


def build_part(group: str, spec: PartSpec):
    """Instantiate the registered kind with the spec's parameters."""
    table = _REGISTRIES[group]
    if spec.kind not in table:
        raise ConfigError(f"unknown {group} kind {spec.kind!r} (registered: {sorted(table)})")
    params = dict(spec.params)
    # a nested position encoding is itself a part
    if isinstance(params.get("position_encoding"), PartSpec):
        params["position_encoding"] = build_part("position_encoding", params["position_encoding"])
    try:
        return table[spec.kind](**params)
    except TypeError as e:
        raise ConfigError(f"{group} {spec.kind!r}: bad parameters {sorted(params)}: {e}") from e


def registered(group: str):
    return sorted(_REGISTRIES[group])
