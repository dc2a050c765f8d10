"""An architecture from outside the package (``tests/toy_arch.py``: a mixer with state of its
own, a windowed group, a layer run three times, a shared cache) goes through the same entry
points as Llama: the random-weights mode writes its folder, the registry reads its config.json,
``Engine.generate`` produces its greedy streams with its stop token.  CPU, with the plain torch
statements of the kernels (``ref_ops``); the GPU versions are in ``test_gpu_parts.py``."""
import copy
import json

import torch

from ref_ops import RefOps
from toy_arch import ToyConfig, plain_toy_forward, plain_toy_greedy
from zllm_b200 import Engine, EngineConfig, ModelRunner, SamplingParams, StepEntry
from zllm_b200.config import architecture_of
from zllm_b200.weights import write_random_model

import plain_llama as P


def toy_folder(tmp_path, seed=4):
    d = write_random_model(tmp_path / "toy", ToyConfig(), seed, "float32", std=0.2, norm_std=0.1)
    return d, P.read_safetensors(d / "model.safetensors")


def test_registry_reads_the_plugins_config_json(tmp_path):
    d, w = toy_folder(tmp_path)
    raw = json.loads((d / "config.json").read_text())
    assert raw["architectures"] == ["ToyHybridForCausalLM"]
    arch = architecture_of(raw)
    spec = arch.build_spec(arch.read_config(raw))
    assert spec.vocab_size == 300 and spec.stop_token_ids == (299,) and "l1.proj" in w


def test_toy_architecture_generates_through_the_engine(tmp_path):
    d, w = toy_folder(tmp_path)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 299, (n,), generator=g).tolist() for n in (5, 23, 2)]
    want = [plain_toy_greedy(w, p, 12) for p in prompts]
    # a stop token taken from the middle of the second stream: emitted, then nothing more
    stop = want[1][5]
    want_stop = [plain_toy_greedy(w, p, 12, stop=(stop,)) for p in prompts]
    assert len(want_stop[1]) <= 6
    eng = Engine(str(d), ops=RefOps(), dtype="float32", device="cpu", cuda_graphs=False, block_size=4, num_blocks=60,
                 max_num_seqs=3, max_num_batched_tokens=16)
    assert eng.generate(prompts, SamplingParams.greedy(max_tokens=12)) == want
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=(stop,)))
    assert got == want_stop
    eng.runner.cache.check_integrity()
    assert eng.stats()["free_slots"] == 3 and eng.stats()["free_pages"] == [60, 60]


def test_the_toy_mixers_device_indexed_path_equals_its_host_path(tmp_path):
    """Steps replayed from a graph give a mixer no host-side description: every row is one token,
    requests are known by ``ctx.row_slot`` alone, padding rows have slot -1."""
    d, w = toy_folder(tmp_path)
    def runner():
        return ModelRunner(str(d), ops=RefOps(), engine_config=EngineConfig(
            dtype="float32", device="cpu", cuda_graphs=False, block_size=4, num_blocks=40, max_num_seqs=4,
            max_num_batched_tokens=32))
    a, b = runner(), runner()
    toks = [[7, 8, 9, 10, 11], [20, 21, 22]]
    for r in (a, b):
        s0, s1, s2 = r.admit(), r.admit(), r.admit()
        r.release(s1)
        r.step([StepEntry(s0, toks[0][:4], ()), StepEntry(s2, toks[1][:2], ())])
    ents = [StepEntry(2, (toks[1][2],), (0,)), StepEntry(0, (toks[0][4],), (0,))]
    la = a.step(ents).clone()                                   # host path: entries are known
    # device path: the same step with the entries hidden and two padding rows behind them
    from zllm_b200.engine.batch import fill_step, make_context
    starts = b._prepare(ents)
    T, R, nd, plans, mc = fill_step(b.buffers, ents, starts, pad_rows=4)
    b.buffers.upload()
    b.cache.sync_tables()
    ctx = make_context(b.buffers, T, R, nd, plans, mc, b.ws)
    assert ctx.entries is None
    lb = b._forward(ctx).clone()
    assert T == 4 and float((la - lb).abs().max()) < 1e-5      # (the products see other row counts)
    assert float((la[1] - plain_toy_forward(w, toks[0])[-1]).abs().max()) < 1e-4
    for i in (1, 4):                                            # the state of the two stateful run entries
        assert float((a.cache.view(i).state - b.cache.view(i).state).abs().max()) < 1e-5
        assert float(b.cache.view(i).state[1].abs().max()) == 0 and float(b.cache.view(i).state[0, -1]) == 5.0
