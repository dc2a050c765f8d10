"""Each part alone against the plain functions, and the generality of the assembly: a toy
mixer with state of its own, defined HERE, is registered, built into a model beside attention
layers (one with a window), run in an order that names a layer twice and lets an entry read
another entry's cache, and stepped in portions -- without a change to the framework's files.
A second toy model does the same for a feed-forward with routing (three experts, the best one
per row, router logits in 32-bit) and for another position encoding (a learned table added to
the embedding output, attention without rotation)."""
import math
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu

import plain_llama as P
from gpu_util import DEV, make_cache, make_ctx
from zllm_b200 import EngineConfig, ModelRunner, StepEntry
from zllm_b200.config import register_architecture
from zllm_b200.models.decoder import Runtime
from zllm_b200.parts import (FeedForward, KVCacheSpec, LayerSpec, Mixer, ModelSpec, PartSpec, PositionEncoding, RunEntry,
                             StateSpec, WeightSpec, build_part, register_feed_forward, register_mixer,
                             register_position_encoding)
from zllm_b200.parts.feedforward import interleave_gate_up


def runtime(dtype):
    from zllm_b200.kernels.ops import CudaOps
    ops = CudaOps(DEV)
    ops.configure(dtype)
    return Runtime(dtype, torch.device(DEV), ops)


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


# bounds relative to the largest magnitude of the expected output
TOL = {torch.float32: 2e-5, torch.bfloat16: 0.02}


def close(got, want, dtype, factor=1.0):
    err = float((got.float().cpu() - want).abs().max())
    return err <= TOL[dtype] * factor * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    rt = runtime(dtype)
    part = build_part("norm", PartSpec("rmsnorm", {"size": 200, "eps": 1e-3}))
    part.bind(rt)
    w = 1 + rnd((200,), 1, 0.2)
    part.load({"weight": w.to(DEV)})                    # stored in 32-bit: stays 32-bit
    x = rnd((9, 200), 2, 4.0)
    out = torch.empty(9, 200, dtype=dtype, device=DEV)
    part.forward(x.to(DEV), out, None)
    assert close(out, P.rmsnorm(x, w, 1e-3), dtype)


def test_rotary_part_tables():
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    part = build_part("position_encoding", PartSpec("rotary", {"rot_dim": 32, "theta": 500000.0, "max_position": 300,
                                                                "scaling": sc}))
    part.bind(runtime(torch.float32))
    t = part.rotary()
    cos, sin = P.rope_tables(P.rope_inv_freq(32, 500000.0, sc), torch.arange(300))
    assert float((t.cos.cpu() - cos).abs().max()) < 1e-6 and float((t.sin.cpu() - sin).abs().max()) < 1e-6
    assert t.rot_dim == 32 and not t.interleaved
    explicit = build_part("position_encoding", PartSpec("rotary", {"rot_dim": 8, "theta": 10000.0, "max_position": 4,
                                                                    "freq_factors": [1.0, 2.0, 0.0, 4.0]}))
    base = P.rope_inv_freq(8, 10000.0, None)
    assert torch.allclose(explicit.inv_freq, base / torch.tensor([1.0, 2.0, 1.0, 4.0]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,I", [(72, 200), (96, 100)])          # I = 100: no multiple of 8, unfused path
def test_swiglu_part(dtype, H, I):
    rt = runtime(dtype)
    part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}))
    part.bind(rt)
    wg, wu, wd = (rnd(s, i, 0.1).to(dtype) for i, s in enumerate([(I, H), (I, H), (H, I)]))
    part.load({"gate_proj": wg.to(DEV), "up_proj": wu.to(DEV), "down_proj": wd.to(DEV)})
    cm = make_cache(1, 16, 4, 8, 1, 32, dtype)
    ctx = make_ctx(cm, [(cm.admit(), 11)])
    h = rnd((11, H), 5).to(dtype)
    res = rnd((11, H), 6)
    out = res.clone().to(DEV)
    part.forward(h.to(DEV), out, ctx)
    want = res + P.swiglu_mlp(h.float(), wg.float(), wu.float(), wd.float())
    assert close(out, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,H,window", [(4, 2, 16, 72, None), (8, 2, 64, 128, None), (3, 1, 32, 96, 9)])
def test_attention_part_whole_and_in_portions(dtype, nq, nkv, hd, H, window):
    rt = runtime(dtype)
    rot = PartSpec("rotary", {"rot_dim": hd, "theta": 10000.0, "max_position": 128})
    part = build_part("mixer", PartSpec("paged_attention", {"hidden_size": H, "n_heads": nq, "n_kv_heads": nkv,
                                                            "head_dim": hd, "position_encoding": rot, "window": window}))
    part.bind(rt)
    assert part.cache_spec() == KVCacheSpec(nkv, hd, window)
    ws = {k: rnd(s.shape, i, 0.15).to(dtype) for i, (k, s) in enumerate(part.weight_specs().items())}
    part.load({k: v.to(DEV) for k, v in ws.items()})
    T = 50
    h = rnd((T, H), 9).to(dtype)
    # plain
    f = {k: v.float() for k, v in ws.items()}
    pos = torch.arange(T)
    cos, sin = P.rope_tables(P.rope_inv_freq(hd, 10000.0, None), pos)
    q = P.apply_rope((h.float() @ f["q_proj"].T).reshape(T, nq, hd), cos, sin, False)
    k = P.apply_rope((h.float() @ f["k_proj"].T).reshape(T, nkv, hd), cos, sin, False)
    v = (h.float() @ f["v_proj"].T).reshape(T, nkv, hd)
    want = P.causal_attention(q, k, v, nq, nkv, pos, window) @ f["o_proj"].T
    for cuts in ([50], [7, 1, 30, 2, 10]):
        cm = make_cache(nkv, hd, 8, 20, 1, 128, dtype, window)
        s = cm.admit()
        got, r = [], 0
        for n in cuts:
            ctx = make_ctx(cm, [(s, n)])
            res = torch.zeros(n, H, device=DEV)
            part.forward(h[r:r + n].to(DEV), res, ctx, cm.view(0))
            got.append(res.cpu())
            r += n
        assert close(torch.cat(got), want, dtype), cuts


# ------------------------------------------------------------------------------------------
# a toy mixer with per-request state of fixed size, defined in the test
# ------------------------------------------------------------------------------------------

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


@dataclass
class ToyConfig:
    architecture: str = "ToyHybridForCausalLM"
    H: int = 64
    V: int = 300


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
    return ModelSpec("ToyHybridForCausalLM", c.V, c.H, 256, layers, order, norm, "emb", {"weight": "fn"}, None)


register_architecture("ToyHybridForCausalLM", lambda d: ToyConfig(**d), build_toy_spec)


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


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    r = ModelRunner(config=ToyConfig(), seed=4, engine_config=EngineConfig(
        dtype="float32", block_size=4, num_blocks=40, max_num_seqs=3, max_num_batched_tokens=128, cuda_graphs=False))
    cm = r.cache
    # groups: full attention (entries 0 and 3), windowed attention (entry 2); state for entries 1 and 4;
    # entry 5 reads entry 0's cache and owns none
    assert [(g.window, g.entries) for g in cm.groups] == [(None, [0, 3]), (12, [2])]
    assert sorted(cm.state) == [1, 4] and cm.view(5) is None
    w = {}
    for name in r.model.expected_tensors():
        pass
    # collect the weights the runner drew, by their names
    exp = r.model.expected_tensors()
    from zllm_b200.weights.random_init import random_tensor
    w = {n: random_tensor(n, s, 4, torch.float32, "cpu") for n, s in exp.items()}
    g = torch.Generator().manual_seed(1)
    ta = torch.randint(0, 300, (60,), generator=g).tolist()
    tb = torch.randint(0, 300, (23,), generator=g).tolist()
    ref_a, ref_b = plain_toy_forward(w, ta), plain_toy_forward(w, tb)
    sa, sb = r.admit(), r.admit()
    got_a, got_b = [], []
    ia = ib = 0
    for na, nb in ((7, 2), (1, 1), (20, 0), (2, 15), (30, 5)):
        ents = []
        if na:
            ents.append(StepEntry(sa, ta[ia:ia + na], tuple(range(na))))
        if nb:
            ents.append(StepEntry(sb, tb[ib:ib + nb], tuple(range(nb))))
        lg = r.step(ents).cpu()
        got_a.append(lg[:na]); got_b.append(lg[na:])
        ia += na; ib += nb
        cm.check_integrity()
    assert float((torch.cat(got_a) - ref_a).abs().max()) < 1e-4
    assert float((torch.cat(got_b) - ref_b).abs().max()) < 1e-4
    # the windowed group gave pages back during the request; the full group did not
    assert cm.groups[1].pool.n_free() > cm.groups[0].pool.n_free()
    r.release(sa)
    # a new request in the freed slot starts from zero state
    sc = r.admit()
    assert sc == sa
    lg = r.step([StepEntry(sc, tb, tuple(range(23)))]).cpu()
    assert float((lg - ref_b).abs().max()) < 1e-4
    r.release(sb); r.release(sc)
    assert cm.free_pages() == [40, 40]


# ------------------------------------------------------------------------------------------
# a toy feed-forward with routing and a toy position encoding, defined in the test
# ------------------------------------------------------------------------------------------

@register_feed_forward("toy_best_expert")
class BestExpert(FeedForward):
    """out = p_e * down_e(relu(up_e h)^2) for the expert e with the largest router logit, p its
    softmax probability; router logits and probabilities in float32."""

    def __init__(self, hidden_size, intermediate_size, n_experts):
        self.H, self.I, self.E = hidden_size, intermediate_size, n_experts

    def weight_specs(self):
        d = {"router": WeightSpec((self.E, self.H), "vector", ("normal", 0.5))}
        for e in range(self.E):
            d[f"up{e}"] = WeightSpec((self.I, self.H), "matrix", ("normal", 0.05))
            d[f"down{e}"] = WeightSpec((self.H, self.I), "matrix", ("normal", 0.05))
        return d

    def forward(self, h, residual, ctx):
        logits = h.float() @ self.router.float().T
        prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
        for e in range(self.E):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel() == 0:
                continue
            up = torch.empty((rows.numel(), self.I), dtype=self.rt.dtype, device=h.device)
            self.rt.ops.linear(h[rows].contiguous(), getattr(self, f"up{e}"), up, "store")
            act = (torch.relu(up.float()) ** 2).to(self.rt.dtype)
            y = torch.zeros((rows.numel(), self.H), dtype=torch.float32, device=h.device)
            self.rt.ops.linear(act, getattr(self, f"down{e}"), y, "add")
            residual[rows] += prob[rows, None] * y


@register_position_encoding("toy_learned_absolute")
class LearnedAbsolute(PositionEncoding):
    """x_t += table[position_t] on the embedding output."""

    def __init__(self, hidden_size, max_position):
        self.H, self.n = hidden_size, max_position

    def weight_specs(self):
        return {"table": WeightSpec((self.n, self.H), "embedding", ("normal", 0.3))}

    def on_embedding(self, x, ctx):
        x += self.table[ctx.positions.long()].float()


@dataclass
class ToyRoutedConfig:
    architecture: str = "ToyRoutedForCausalLM"
    H: int = 48
    V: int = 200


def build_routed_spec(c: ToyRoutedConfig) -> ModelSpec:
    attn = PartSpec("paged_attention", {"hidden_size": c.H, "n_heads": 3, "n_kv_heads": 3, "head_dim": 16,
                                        "position_encoding": None, "window": None})
    norm = PartSpec("rmsnorm", {"size": c.H, "eps": 1e-6})
    routed = PartSpec("toy_best_expert", {"hidden_size": c.H, "intermediate_size": 40, "n_experts": 3})
    dense = PartSpec("swiglu", {"hidden_size": c.H, "intermediate_size": 72})
    qkvo = {f"mixer.{k}": k for k in ("q_proj", "k_proj", "v_proj", "o_proj")}
    def names(i, ffn_names):
        d = {"norm1.weight": f"l{i}.n1", "norm2.weight": f"l{i}.n2"}
        d.update({k: f"l{i}.{v}" for k, v in qkvo.items()})
        d.update({f"ffn.{k}": f"l{i}.{k}" for k in ffn_names})
        return d
    experts = ["router"] + [f"{w}{e}" for e in range(3) for w in ("up", "down")]
    layers = [LayerSpec(attn, routed, norm, norm, "pre_norm", names(0, experts)),
              LayerSpec(attn, dense, norm, norm, "pre_norm", names(1, ("gate_proj", "up_proj", "down_proj")))]
    return ModelSpec("ToyRoutedForCausalLM", c.V, c.H, 128, layers, [RunEntry(0), RunEntry(1)], norm, "emb", {"weight": "fn"},
                     "head", embedding_position=PartSpec("toy_learned_absolute", {"hidden_size": c.H, "max_position": 128}),
                     embedding_position_names={"table": "pos"})


register_architecture("ToyRoutedForCausalLM", lambda d: ToyRoutedConfig(**d), build_routed_spec)


def plain_routed_forward(w, tokens):
    T = len(tokens)
    pos = torch.arange(T)
    x = w["emb"][torch.tensor(tokens)] + w["pos"][pos]
    for i in range(2):
        h = P.rmsnorm(x, w[f"l{i}.n1"], 1e-6)
        q, k, v = ((h @ w[f"l{i}.{n}_proj"].T).reshape(T, 3, 16) for n in "qkv")
        x = x + P.causal_attention(q, k, v, 3, 3, pos, None) @ w[f"l{i}.o_proj"].T
        h = P.rmsnorm(x, w[f"l{i}.n2"], 1e-6)
        if i == 0:
            prob, choice = torch.softmax(h @ w["l0.router"].T, dim=-1).max(dim=-1)
            y = torch.stack([torch.relu(h[t] @ w[f"l0.up{int(choice[t])}"].T) ** 2 @ w[f"l0.down{int(choice[t])}"].T
                             for t in range(T)])
            x = x + prob[:, None] * y
        else:
            x = x + P.swiglu_mlp(h, w["l1.gate_proj"], w["l1.up_proj"], w["l1.down_proj"])
    return P.rmsnorm(x, w["fn"], 1e-6) @ w["head"].T


def test_toy_routed_feed_forward_and_learned_positions_are_registered_built_and_stepped():
    r = ModelRunner(config=ToyRoutedConfig(), seed=6, engine_config=EngineConfig(
        dtype="float32", block_size=8, num_blocks=24, max_num_seqs=3, max_num_batched_tokens=96, cuda_graphs=False))
    from zllm_b200.weights.random_init import random_tensor
    w = {n: random_tensor(n, s, 6, torch.float32, "cpu") for n, s in r.model.expected_tensors().items()}
    assert w["pos"].shape == (128, 48) and w["l0.router"].shape == (3, 48)
    g = torch.Generator().manual_seed(2)
    ta = torch.randint(0, 200, (50,), generator=g).tolist()
    tb = torch.randint(0, 200, (31,), generator=g).tolist()
    ref_a, ref_b = plain_routed_forward(w, ta), plain_routed_forward(w, tb)
    sa, sb = r.admit(), r.admit()
    got_a, got_b = [], []
    ia = ib = 0
    for na, nb in ((9, 1), (1, 1), (25, 2), (2, 20), (13, 7)):
        ents = []
        if na:
            ents.append(StepEntry(sa, ta[ia:ia + na], tuple(range(na))))
        if nb:
            ents.append(StepEntry(sb, tb[ib:ib + nb], tuple(range(nb))))
        lg = r.step(ents).cpu()
        got_a.append(lg[:na]); got_b.append(lg[na:])
        ia += na; ib += nb
    assert float((torch.cat(got_a) - ref_a).abs().max()) < 2e-4
    assert float((torch.cat(got_b) - ref_b).abs().max()) < 2e-4
    # the position table matters: the same tokens one position later give other logits
    r.release(sa); r.release(sb)
    sc = r.admit()
    shifted = r.step([StepEntry(sc, [ta[0]] + ta[:8], tuple(range(9)))]).cpu()
    assert float((shifted[1:] - ref_a[:8]).abs().max()) > 1e-2
