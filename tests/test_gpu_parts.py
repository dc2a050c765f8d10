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
# a toy architecture with a stateful mixer: defined in tests/toy_arch.py, a plug-in module of the
# test-suite (so that the command line programs can load it too), not in the package
# ------------------------------------------------------------------------------------------
from toy_arch import ToyConfig, plain_toy_forward, plain_toy_greedy          # noqa: E402  (registers the architecture)


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    r = ModelRunner(config=ToyConfig(), seed=4, engine_config=EngineConfig(
        dtype="float32", block_size=4, num_blocks=40, max_num_seqs=3, max_num_batched_tokens=128, cuda_graphs=False))
    cm = r.cache
    # groups: full attention (entries 0 and 3), windowed attention (entry 2); state for entries 1 and 4;
    # entry 5 reads entry 0's cache and owns none
    assert [(g.window, g.entries) for g in cm.groups] == [(None, [0, 3]), (12, [2])]
    assert sorted(cm.state) == [1, 4] and cm.view(5) is None
    # the weights the runner drew, by their names
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


@pytest.mark.parametrize("graphs", [True, False])
def test_toy_architecture_generates_through_the_engine(tmp_path, graphs):
    """The toy architecture through ``Engine.generate``: greedy streams with a stop token, four
    requests through three slots.  With graphs on, its stateful mixer runs inside captured decode
    graphs (and the run-ahead), where it knows its rows' requests by device-side slots only."""
    from zllm_b200 import Engine, SamplingParams
    from zllm_b200.weights import write_random_model
    d = write_random_model(tmp_path / "toy", ToyConfig(), 4, "float32", std=0.2, norm_std=0.1)
    w = P.read_safetensors(d / "model.safetensors")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 299, (n,), generator=g).tolist() for n in (5, 23, 2, 11)]
    free_run = [plain_toy_greedy(w, p, 14) for p in prompts]
    stop = free_run[1][6]
    want = [plain_toy_greedy(w, p, 14, stop=(stop,)) for p in prompts]
    eng = Engine(str(d), dtype="float32", block_size=4, num_blocks=80, max_num_seqs=3, max_num_batched_tokens=24,
                 cuda_graphs=graphs)
    assert eng.generate(prompts, SamplingParams.greedy(max_tokens=14)) == free_run
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=14, stop_token_ids=(stop,)))
    assert got == want
    if graphs:
        assert eng.runner._graphs and all(g["graph"] is not None for g in eng.runner._graphs.values())
    eng.runner.cache.check_integrity()
    assert eng.stats()["free_slots"] == 3 and eng.stats()["free_pages"] == [80, 80]


def test_toy_architecture_through_trace_run_as_a_plugin(tmp_path):
    """``bin/trace_run`` on the toy architecture's model folder: the program learns the architecture
    from the plug-in module named in ZLLM_PLUGINS, nothing of the framework's files changes."""
    import os
    import traces as TR
    from zllm_b200.weights import write_random_model
    d = write_random_model(tmp_path / "toy", ToyConfig(), 4, "float32", std=0.2, norm_std=0.1)
    w = P.read_safetensors(d / "model.safetensors")
    g = torch.Generator().manual_seed(5)
    reqs = [(f"r{i}", torch.randint(0, 300, (n,), generator=g).tolist()) for i, n in enumerate((9, 40, 3, 26))]
    ref = {rid: plain_toy_forward(w, toks) for rid, toks in reqs}
    steps = TR.family_whole(reqs, "w.") + TR.family_tail(reqs, 8, "t.") + TR.family_portions(reqs, prefix="p.") \
        + TR.family_mixed(reqs, 192, 3, 1, "m.")
    tests_dir = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, ZLLM_PLUGINS="toy_arch",
               PYTHONPATH=tests_dir + os.pathsep + os.environ.get("PYTHONPATH", ""))
    got = TR.replay_program(d, "float32", steps, 192, tmp_path / "out", 300, extra_args=("--block-size", "4"), env=env)
    for prefix in ("w.", "t.", "p.", "m."):
        TR.compare(got, ref, reqs, prefix, 1e-4, 0.0, f"toy {prefix}")
    for rid, toks in reqs:                           # the ways of cutting agree among themselves
        for p_ in range(len(toks)):
            for prefix in ("t.", "p.", "m."):
                assert float((got[("w." + rid, p_)] - got[(prefix + rid, p_)]).abs().max()) < 2e-5


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
