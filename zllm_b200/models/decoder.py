"""A decoder assembled from a ``ModelSpec``: embedding, layers in their run
order, final norm, output head.

Order of one forward as in zllm src/backend/candle/quantized_llama_fork.rs:920-987:
embed (935), layers (936-968), final norm (971), select the wanted rows (972),
head (980).  The reference computes logits only for the last row of a call;
here only for the rows the batch asks for.  A missing head tensor means the
head is the embedding table (fork.rs:761-764).
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..errors import ConfigError
from ..parts.base import ModelSpec, PartSpec, WeightSpec, build_part, _REGISTRIES
from ..parts.block import Layer


@dataclass
class Runtime:
    """What parts get at bind time: compute dtype, device and the kernel table."""

    dtype: torch.dtype
    device: torch.device
    ops: object


def _build_layers(spec: ModelSpec):
    memo: Dict[str, object] = {}

    def build(group, pspec: PartSpec):
        params = dict(pspec.params)
        pe = params.get("position_encoding")
        if isinstance(pe, PartSpec):
            key = repr((pe.kind, sorted(pe.params.items(), key=lambda kv: kv[0])))
            if key not in memo:
                memo[key] = build_part("position_encoding", pe)
            params["position_encoding"] = memo[key]
        return build_part(group, PartSpec(pspec.kind, params))

    layers = []
    for ls in spec.layers:
        if ls.arrangement not in _REGISTRIES["arrangement"]:
            raise ConfigError(f"unknown arrangement {ls.arrangement!r}")
        layers.append(Layer(build("norm", ls.norm1), build("mixer", ls.mixer), build("norm", ls.norm2),
                            build("feed_forward", ls.ffn), _REGISTRIES["arrangement"][ls.arrangement]))
    final_norm = build("norm", spec.final_norm)
    position = build("position_encoding", spec.embedding_position) if spec.embedding_position is not None else None
    return layers, final_norm, position


def _named_specs(spec: ModelSpec, layers: List[Layer], final_norm, position=None) -> Dict[str, WeightSpec]:
    out: Dict[str, WeightSpec] = {}
    out[spec.embedding_name] = WeightSpec((spec.vocab_size, spec.hidden_size), "embedding", ("normal", spec.init_std))
    if position is not None:
        for local, ws in position.weight_specs().items():
            if local not in spec.embedding_position_names:
                raise ConfigError(f"no tensor name given for the embedding position encoding's {local}")
            out[spec.embedding_position_names[local]] = ws
    for li, (ls, layer) in enumerate(zip(spec.layers, layers)):
        for pname, part in layer.parts().items():
            for local, ws in part.weight_specs().items():
                key = f"{pname}.{local}"
                if key not in ls.tensor_names:
                    raise ConfigError(f"layer {li}: no tensor name given for {key}")
                out[ls.tensor_names[key]] = ws
    for local, ws in final_norm.weight_specs().items():
        out[spec.final_norm_names[local]] = ws
    if spec.head_name is not None and not spec.head_optional:
        out[spec.head_name] = _head_spec(spec)
    return out


def _head_spec(spec: ModelSpec) -> WeightSpec:
    return WeightSpec((spec.vocab_size, spec.hidden_size), "matrix", ("normal", spec.init_std))


def optional_tensors(spec: ModelSpec) -> Dict[str, WeightSpec]:
    """Tensors a folder may hold or lack: the output head of a model whose head falls back to the
    embedding table when it is absent."""
    if spec.head_name is not None and spec.head_optional:
        return {spec.head_name: _head_spec(spec)}
    return {}


def required_tensors(spec: ModelSpec) -> Dict[str, WeightSpec]:
    """Every tensor the model folder must hold: name -> shape, role, init."""
    return _named_specs(spec, *_build_layers(spec))


def expected_tensors(spec: ModelSpec) -> Dict[str, WeightSpec]:
    """The tensors the random-weights mode writes: the required ones, and an optional head
    unless the configuration ties it."""
    out = required_tensors(spec)
    if not spec.tie_head:
        out.update(optional_tensors(spec))
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.layers, self.final_norm, self.position = _build_layers(spec)
        for i, e in enumerate(spec.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"run order entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_of is not None and not (0 <= e.cache_of < i and spec.run_order[e.cache_of].cache_of is None):
                raise ConfigError(f"run order entry {i}: cache_of must name an earlier entry that owns its cache")
        for layer in self.layers:
            for part in layer.parts().values():
                part.bind(rt)
        self.final_norm.bind(rt)
        if self.position is not None:
            self.position.bind(rt)
        self.embedding = None
        self.head = None

    # ---- weights -------------------------------------------------------
    def required_tensors(self) -> Dict[str, WeightSpec]:
        return _named_specs(self.spec, self.layers, self.final_norm, self.position)

    def optional_tensors(self) -> Dict[str, WeightSpec]:
        return optional_tensors(self.spec)

    def expected_tensors(self) -> Dict[str, WeightSpec]:
        """Required tensors plus the optional ones the configuration asks for (random mode)."""
        out = self.required_tensors()
        if not self.spec.tie_head:
            out.update(self.optional_tensors())
        return out

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        spec = self.spec
        self.embedding = tensors[spec.embedding_name]
        for ls, layer in zip(spec.layers, self.layers):
            for pname, part in layer.parts().items():
                local = {name: tensors[ls.tensor_names[f"{pname}.{name}"]] for name in part.weight_specs()}
                part.load(local)
        self.final_norm.load({n: tensors[spec.final_norm_names[n]] for n in self.final_norm.weight_specs()})
        if self.position is not None:
            self.position.load({n: tensors[spec.embedding_position_names[n]] for n in self.position.weight_specs()})
        # a head tensor that is there is used; without one the head is the embedding table
        head = tensors.get(spec.head_name) if spec.head_name is not None else None
        if head is None and spec.head_name is not None and not spec.head_optional:
            raise ConfigError(f"the output head {spec.head_name!r} was not given")
        if spec.head_optional and (head is None) != bool(spec.tie_head):
            warnings.warn(f"{spec.architecture}: the configuration says the output head is "
                          f"{'tied' if spec.tie_head else 'untied'}, the weights "
                          f"{'lack' if head is None else 'hold'} {spec.head_name!r}; "
                          f"{'the embedding table' if head is None else 'the stored tensor'} is used")
        self.head = head if head is not None else self.embedding

    # ---- cache needs ---------------------------------------------------
    def cache_needs(self):
        """Per run entry: (cache spec of its mixer or None, cache_of)."""
        return [(self.layers[e.layer].mixer.cache_spec(), e.cache_of) for e in self.spec.run_order]

    def capturable(self) -> bool:
        """True when every part says that a step with prompt portions may be captured as a graph."""
        parts = [p for layer in self.layers for p in layer.parts().values()] + [self.final_norm]
        if self.position is not None:
            parts.append(self.position)
        for p in list(parts):
            pe = getattr(p, "position_encoding", None)
            if pe is not None:
                parts.append(pe)
        return all(getattr(p, "capturable", False) for p in parts)

    def step_planners(self):
        """The planners of the model's parts, each once: callables that write a part's own tables
        for a step into the step buffer (``parts.base.Part.step_planner``)."""
        seen, out = set(), []
        for layer in self.layers:
            for part in layer.parts().values():
                pl = part.step_planner()
                if pl is not None and pl not in seen:
                    seen.add(pl)
                    out.append(pl)
        return tuple(out)

    # ---- one forward over the step's rows ------------------------------
    def forward(self, ctx, cache_views) -> Optional[torch.Tensor]:
        """Runs the rows of ``ctx``; returns float32 logits [R, V] for ``ctx.want_rows`` (None if R == 0)."""
        ops, rt = self.rt.ops, self.rt
        T = ctx.T
        x = ctx.ws.get("residual", (T, self.spec.hidden_size), torch.float32)
        ops.embedding(ctx.token_ids, self.embedding, x)
        if self.position is not None:
            self.position.on_embedding(x, ctx)
        for i, e in enumerate(self.spec.run_order):
            owner = i if e.cache_of is None else e.cache_of
            self.layers[e.layer].run(x, ctx, cache_views[owner], write_cache=e.cache_of is None)
        R = ctx.R
        if R == 0:
            return None
        logits = ctx.ws.get("logits", (R, self.spec.vocab_size), torch.float32, cap=R)
        pro = self.final_norm.as_prologue()
        if pro is not None:
            # a norm that can stand as a product's prologue also takes the wanted rows by index
            ops.linear_normed(x, pro[0], pro[1], self.head, logits, "store", ctx.ws, rows=ctx.want_rows)
        else:
            rows = ctx.ws.get("head_rows", (R, self.spec.hidden_size), torch.float32, cap=R)
            ops.gather_rows(x, ctx.want_rows, rows)
            hn = ctx.ws.get("head_in", (R, self.spec.hidden_size), rt.dtype, cap=R)
            self.final_norm.forward(rows, hn, ctx)
            ops.linear(hn, self.head, logits, "store")
        return logits
