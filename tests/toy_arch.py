"""A toy architecture of the TEST-SUITE, not of the package: a mixer with per-request state of
its own (a running mean), registered and built into a model beside attention layers (one with a
window), run in an order that names a layer twice and lets an entry read another entry's cache.

It lives in a module of its own so that it can be loaded as a plug-in (``ZLLM_PLUGINS=toy_arch``
with ``tests/`` on the path): the Python entry point, the command line and ``bin/trace_run`` then
take its model folders without a change to the framework's files.  It is nobody's model.

The mixer shows what a mixer with state must do to run inside captured decode graphs: a graph
replays with other requests in its rows, so nothing about the step may be read on the host.  In
such a step every row is a single token, ``ctx.entries`` is None, and the request of a row is
``ctx.row_slot`` ON THE DEVICE (-1 for padding rows); the state is read and written with device
indices, by operations on the current stream.
"""
from __future__ import annotations

import os
import sys
from dataclasses import asdict, dataclass

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import plain_llama as P          # noqa: E402
from zllm_b200.config import register_architecture          # noqa: E402
from zllm_b200.parts import (LayerSpec, Mixer, ModelSpec, PartSpec, RunEntry, StateSpec, WeightSpec,          # noqa: E402
                             register_mixer)


@register_mixer("toy_running_mean")
class RunningMean(Mixer):
    """out_t = W * mean(h_0..h_t): the state is the running sum and the count."""

    def __init__(self, hidden_size):
        self.H = hidden_size
        self.proj = None

    def weight_specs(self):
        return {"proj": WeightSpec((self.H, self.H), "matrix", ("normal", 0.05))}

    def cache_spec(self):
        return StateSpec((self.H + 1,), "float32")

    def forward(self, h, residual, ctx, cache, write_cache=True):
        if ctx.entries is None:
            return self._single_tokens(h, residual, ctx, cache)
        r = 0
        for e in ctx.entries:                              # rows of one request are in order
            n = len(e.tokens)
            st = cache.state[e.slot]
            csum = torch.cumsum(h[r:r + n].float(), 0) + st[:self.H]
            cnt = st[self.H] + torch.arange(1, n + 1, device=h.device)
            mean = (csum / cnt[:, None]).to(self.rt.dtype)
            self.rt.ops.linear(mean.contiguous(), self.proj, residual[r:r + n], "add")
            st[:self.H] = csum[-1]
            st[self.H] = cnt[-1]
            r += n

    def _single_tokens(self, h, residual, ctx, cache):
        """Every row is one token of another request (a decode step, possibly a replayed graph):
        the rows' slots are compared on the device; padding rows (slot -1) match no slot, read a
        zero state and write nothing.  Shapes are fixed and nothing is read by the host."""
        S = cache.state                                                    # [slots, H + 1]
        hit = ctx.row_slot[:, None] == torch.arange(S.shape[0], device=h.device, dtype=ctx.row_slot.dtype)[None, :]
        st = (hit[:, :, None] * S[None]).sum(1)                            # each row's state (exact: one term)
        csum = h.float() + st[:, :self.H]
        cnt = st[:, self.H] + 1.0
        mean = (csum / cnt[:, None]).to(self.rt.dtype).contiguous()
        add = torch.zeros_like(residual)
        self.rt.ops.linear(mean, self.proj, add, "add")
        residual += torch.where(hit.any(1)[:, None], add, torch.zeros_like(add))
        new = torch.cat([csum, cnt[:, None]], dim=1)
        upd = (hit.t()[:, :, None] * new[None]).sum(1)                     # a slot is in at most one row
        S.copy_(torch.where(hit.any(0)[:, None], upd, S))


@dataclass
class ToyConfig:
    architecture: str = "ToyHybridForCausalLM"
    H: int = 64
    V: int = 300

    @staticmethod
    def from_dict(d: dict) -> "ToyConfig":
        return ToyConfig(H=int(d["H"]), V=int(d["V"]))

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        return d


def build_toy_spec(c: ToyConfig) -> ModelSpec:
    rot = PartSpec("rotary", {"rot_dim": 16, "theta": 10000.0, "max_position": 256})
    def attn(window):
        return PartSpec("paged_attention", {"hidden_size": c.H, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16,
                                            "position_encoding": rot, "window": window})
    norm = PartSpec("rmsnorm", {"size": c.H, "eps": 1e-5})
    ffn = PartSpec("swiglu", {"hidden_size": c.H, "intermediate_size": 96})
    def names(i, mixer_names):
        d = {"norm1.weight": f"l{i}.n1", "norm2.weight": f"l{i}.n2", "ffn.gate_proj": f"l{i}.g",
             "ffn.up_proj": f"l{i}.u", "ffn.down_proj": f"l{i}.d"}
        d.update({f"mixer.{k}": f"l{i}.{k}" for k in mixer_names})
        return d
    qkvo = ("q_proj", "k_proj", "v_proj", "o_proj")
    layers = [LayerSpec(attn(None), ffn, norm, norm, "pre_norm", names(0, qkvo)),
              LayerSpec(PartSpec("toy_running_mean", {"hidden_size": c.H}), ffn, norm, norm, "pre_norm", names(1, ("proj",))),
              LayerSpec(attn(12), ffn, norm, norm, "pre_norm", names(2, qkvo))]
    # layer 0 runs twice with caches of its own; the last entry runs layer 0 a third time
    # and reads the cache that run entry 0 wrote
    order = [RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(0), RunEntry(1), RunEntry(0, cache_of=0)]
    return ModelSpec("ToyHybridForCausalLM", c.V, c.H, 256, layers, order, norm, "emb", {"weight": "fn"}, None,
                     stop_token_ids=(299,))


register_architecture("ToyHybridForCausalLM", ToyConfig.from_dict, build_toy_spec)


def plain_toy_forward(w, tokens, H=64):
    """Whole-sequence statement of the toy model with the plain functions."""
    T = len(tokens)
    pos = torch.arange(T)
    cos, sin = P.rope_tables(P.rope_inv_freq(16, 10000.0, None), pos)
    x = w["emb"][torch.tensor(tokens)]
    kv0 = None

    def attn(i, h, window, reuse=None):
        q = P.apply_rope((h @ w[f"l{i}.q_proj"].T).reshape(T, 4, 16), cos, sin, False)
        if reuse is None:
            k = P.apply_rope((h @ w[f"l{i}.k_proj"].T).reshape(T, 2, 16), cos, sin, False)
            v = (h @ w[f"l{i}.v_proj"].T).reshape(T, 2, 16)
        else:
            k, v = reuse
        return P.causal_attention(q, k, v, 4, 2, pos, window) @ w[f"l{i}.o_proj"].T, (k, v)

    for e, (layer, cache_of) in enumerate([(0, None), (1, None), (2, None), (0, None), (1, None), (0, 0)]):
        h = P.rmsnorm(x, w[f"l{layer}.n1"], 1e-5)
        if layer == 1:
            mean = torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]
            x = x + mean @ w["l1.proj"].T
        else:
            y, kv = attn(layer, h, 12 if layer == 2 else None, kv0 if cache_of is not None else None)
            if e == 0:
                kv0 = kv
            x = x + y
        h = P.rmsnorm(x, w[f"l{layer}.n2"], 1e-5)
        x = x + P.swiglu_mlp(h, w[f"l{layer}.g"], w[f"l{layer}.u"], w[f"l{layer}.d"])
    return P.rmsnorm(x, w["fn"], 1e-5) @ w["emb"].T


def plain_toy_greedy(w, prompt, n_new, stop=()):
    """The toy model's greedy stream by whole-sequence recompute; a stop token is emitted and ends it."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        t = P.argmax_lowest(plain_toy_forward(w, toks)[-1])
        out.append(t)
        toks.append(t)
        if t in stop:
            break
    return out
