"""Generation through the Python entry point and the command line, on the GPU."""
import json
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

import plain_llama as P
import traces as TR
from configs import GEN_STD, TINY, make_model_dir, random_prompt
from gpu_util import BF16_GAP_OF_SCALE, bf16_bound, check_greedy_stream, observe
from zllm_b200 import Engine, EngineConfig, ModelRunner, SamplingParams, Session, StepEntry


def plain_forward(cfg, w):
    return lambda toks: P.forward_all_positions(cfg, w, toks)


def gumbel_scores(logits, temperature, seed):
    """logit_i / temp - log(-log u_i) for the whole vocabulary, u_i as ``P.rand01`` (vectorised;
    shaders.rs:805-836)."""
    import numpy as np
    def h32(x):
        x = x.astype(np.uint64) & 0xFFFFFFFF
        x ^= x >> 16
        x = (x * 0x7FEB352D) & 0xFFFFFFFF
        x ^= x >> 15
        x = (x * 0x846CA68B) & 0xFFFFFFFF
        x ^= x >> 16
        return x
    i = np.arange(logits.numel(), dtype=np.uint64)
    r = h32(np.uint64(seed & 0xFFFFFFFF) ^ h32(i))
    u = torch.from_numpy((((r >> 8).astype(np.float64)) + 0.5) / 16777216.0).float()
    return logits.float() / temperature - torch.log(-torch.log(u))


def check_gumbel_stream(cfg, w, prompt, got, temperature, seed, dtype, name, what):
    """A temperature-sampled stream, teacher-forced on itself: token n must maximise the plain
    logits / temp + Gumbel noise of seed n; in bfloat16 within a near-tie's gap of the best."""
    lg = P.forward_all_positions(cfg, w, list(prompt) + list(got[:-1]))[len(prompt) - 1:]
    for n, t in enumerate(got):
        sc = gumbel_scores(lg[n], temperature, P.step_seed(seed, n))
        best = int(sc.argmax())
        if t == best:
            continue
        assert dtype != "float32", f"{what}: token {n} is {t}, plain samples {best}"
        gap = float(sc[best] - sc[t]) * temperature
        scale = float(lg[n].abs().max())
        observe(f"near-tie gap {what}", gap, scale, BF16_GAP_OF_SCALE)
        assert gap <= BF16_GAP_OF_SCALE * scale, f"{what}: token {n}: gap {gap:.3e}"


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(tmp_path, name, dtype):
    """Sharper logits (larger weights) so that greedy choices are not rounding ties."""
    d = make_model_dir(tmp_path, name, dtype, std=GEN_STD[name])
    cfg, w = P.read_model_dir(d)
    V = cfg["vocab_size"]
    prompts = [random_prompt(V, n, 50 + n) for n in (5, 17, 33)]
    want = [P.greedy_generate(cfg, w, p, 16) for p in prompts]
    for nb, budget in ((64, 512), (9, 7)):
        eng = Engine(str(d), dtype=dtype, block_size=TINY[name][1], num_blocks=nb * 16 // TINY[name][1],
                     max_num_seqs=4, max_num_batched_tokens=budget)
        out = eng.generate(prompts, SamplingParams.greedy(max_tokens=16))
        if dtype == "float32":
            assert out == want
        for o, p in zip(out, prompts):
            # every token is the plain argmax given the stream so far; bfloat16 may take a near-tie
            check_greedy_stream(plain_forward(cfg, w), p, o, dtype, 16, what=f"tiny {name} greedy")
        assert eng.stats()["free_pages"] == [nb * 16 // TINY[name][1]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_and_topk_sampling(tmp_path, dtype):
    d = make_model_dir(tmp_path, "B", dtype, std=GEN_STD["B"])
    prompts = [random_prompt(1000, n, 70 + n) for n in (3, 30, 12, 40)]
    params = [SamplingParams.with_temperature(0.8, seed=100 + i, max_tokens=24) for i in range(3)]
    params.append(SamplingParams(temperature=0.9, top_k=5, top_p=0.9, seed=7, max_tokens=24))

    def run(nb, budget):
        eng = Engine(str(d), dtype=dtype, block_size=8, num_blocks=nb, max_num_seqs=4, max_num_batched_tokens=budget)
        return eng.generate(prompts, params), eng.stats()

    cfg, w = P.read_model_dir(d)
    a, _ = run(64, 256)
    b, st = run(17, 11)                          # few pages: preemption and recompute in between
    assert st["preemptions"] > 0                 # requests were resumed by prefilling prompt ++ produced tokens
    assert a == run(64, 256)[0]                  # same seeds, same tokens
    if dtype == "float32":
        assert a == b
    for out, how in ((a, "roomy"), (b, "preempted")):
        # each stream against the plain implementation, teacher-forced on itself: what a resumed
        # request produces after its recompute is held to the same rule as everything else
        for i in range(3):
            assert len(out[i]) == 24
            check_gumbel_stream(cfg, w, prompts[i], out[i], 0.8, 100 + i, dtype, "B", f"tiny B sampled {how}")
        toks = list(prompts[3])
        for n, t in enumerate(out[3]):           # top-k 5: the token is one of the plain top candidates
            lg = P.forward_all_positions(cfg, w, toks)[-1]
            assert t in P.topk_desc(lg, 5 if dtype == "float32" else 7)[1], (how, n)
            toks.append(t)
    greedy = SamplingParams(temperature=0.0, seed=5, max_tokens=8)
    eng = Engine(str(d), dtype=dtype, block_size=8, max_num_seqs=2)
    g1 = eng.generate(prompts[:1], greedy)
    greedy2 = SamplingParams(temperature=0.0, seed=99, max_tokens=8)
    assert eng.generate(prompts[:1], greedy2) == g1          # temperature 0: the seed does not matter


def test_topk_topp_sampling_on_the_device_equals_the_host_path(tmp_path):
    """Decode steps draw top-k / top-p tokens inside the captured graph (and run ahead of the host);
    with graphs off the host draws from the same candidates.  Same seeds: the same streams, and
    the first tokens are what the plain implementation samples."""
    d = make_model_dir(tmp_path, "B", "float32", std=0.2)
    cfg, w = P.read_model_dir(d)
    prompts = [random_prompt(1000, n, 90 + n) for n in (4, 21, 9, 33, 2)]
    params = [SamplingParams(temperature=0.9, top_k=5, top_p=0.9, seed=7, max_tokens=30),
              SamplingParams(temperature=1.2, top_k=0, top_p=0.8, seed=8, max_tokens=30),
              SamplingParams(temperature=0.7, top_k=40, top_p=1.0, seed=9, max_tokens=30),
              SamplingParams.with_temperature(0.8, seed=10, max_tokens=30),
              SamplingParams.greedy(max_tokens=30)]
    outs = []
    for graphs in (True, False):
        eng = Engine(str(d), dtype="float32", block_size=8, num_blocks=64, max_num_seqs=8, cuda_graphs=graphs)
        assert eng._device_pool == graphs
        outs.append(eng.generate(prompts, params))
        if graphs:
            assert any(k[2] for k in eng.runner._graphs)     # a graph with the draw in it was captured
    assert outs[0] == outs[1]
    toks = list(prompts[0])
    for n in range(3):
        v, i = P.topk_desc(P.forward_all_positions(cfg, w, toks)[-1], 64)
        t = P.sample_topk(v, i, 0.9, 5, 0.9, P.step_seed(7, n))
        assert t == outs[0][0][n]
        toks.append(t)


def test_warm_up_captures_every_bucket(tmp_path):
    d = make_model_dir(tmp_path, "C", "bfloat16")
    eng = Engine(str(d), dtype="bfloat16", max_num_seqs=5, max_model_len=600, num_blocks=64)
    n = eng.warm_up()
    assert n == 4 * 3 and eng.warm_up() == 0           # rows 1, 2, 4, 8 x splits 1, 2, 4
    assert eng.warm_up(max_batch=2, max_context=200, sampling=True) == 2      # the variants with the draw in them
    before = set(eng.runner._graphs)
    out = eng.generate([random_prompt(1536, 300, 1), random_prompt(1536, 5, 2)], SamplingParams.greedy(max_tokens=30))
    assert set(eng.runner._graphs) == before and len(out[0]) == 30


def test_small_graphs_stay_valid_when_the_batch_has_grown(tmp_path):
    """Decode graphs of a small batch are captured first, then a larger batch makes the scratch
    buffers grow, then the small batch runs again through its old graphs (which hold the addresses
    of the old buffers) while the larger batch's buffers are in use: every stream must still be the
    plain implementation's.  float32, so the streams are exact."""
    d = make_model_dir(tmp_path, "A", "float32", std=0.3)
    cfg, w = P.read_model_dir(d)
    V = cfg["vocab_size"]
    prompts = [random_prompt(V, 4 + 3 * i, 70 + i) for i in range(7)]
    # the first two requests run long, the others end early: the batch is 2, then 7, then 2 again
    lens = [40, 40, 6, 6, 6, 6, 6]
    want = [P.greedy_generate(cfg, w, p, n) for p, n in zip(prompts, lens)]
    eng = Engine(str(d), dtype="float32", block_size=TINY["A"][1], num_blocks=64 * 16 // TINY["A"][1], max_num_seqs=8,
                 max_num_batched_tokens=64)
    got = {}
    ids = [eng.add_request(p, SamplingParams.greedy(max_tokens=n)) for p, n in zip(prompts[:2], lens[:2])]
    for _ in range(6):                                        # batch of 2: graphs of the small bucket
        for rid, tok, done in eng.step():
            got.setdefault(rid, []).append(tok)
    ids += [eng.add_request(p, SamplingParams.greedy(max_tokens=n)) for p, n in zip(prompts[2:], lens[2:])]
    while eng.has_unfinished():
        for rid, tok, done in eng.step():
            got.setdefault(rid, []).append(tok)
    assert [got[i] for i in ids] == want
    assert len({k[0] for k in eng.runner._graphs}) >= 2      # at least two batch buckets were captured


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_requests_through_few_slots_and_few_pages(tmp_path, dtype):
    """Thirty requests of random lengths through five slots and so few pages that requests are
    preempted: batches grow and shrink, slots and pages change hands, decode graphs of every size
    run in turn between mixed steps.  float32: every stream must be the plain implementation's;
    bfloat16: every token the plain argmax given its own stream, or a near-tie."""
    import random
    d = make_model_dir(tmp_path, "B", dtype, std=GEN_STD["B"])
    cfg, w = P.read_model_dir(d)
    V = cfg["vocab_size"]
    rng = random.Random(5)
    prompts = [random_prompt(V, rng.randint(1, 40), 300 + i) for i in range(30)]
    lens = [rng.randint(1, 24) for _ in prompts]
    want = [P.greedy_generate(cfg, w, p, n) for p, n in zip(prompts, lens)]
    bs = TINY["B"][1]
    eng = Engine(str(d), dtype=dtype, block_size=bs, num_blocks=-(-150 // bs), max_num_seqs=5, max_num_batched_tokens=48)
    got = {}
    ids = []
    pending = list(zip(prompts, lens))
    while pending or eng.has_unfinished():
        for _ in range(rng.randint(0, 3)):                   # requests arrive while others run
            if pending:
                p, n = pending.pop(0)
                ids.append(eng.add_request(p, SamplingParams.greedy(max_tokens=n)))
        for rid, tok, done in eng.step():
            got.setdefault(rid, []).append(tok)
    if dtype == "float32":
        assert [got[i] for i in ids] == want
    for i, p, n in zip(ids, prompts, lens):
        check_greedy_stream(plain_forward(cfg, w), p, got[i], dtype, n, what="tiny B many requests")
    st = eng.stats()
    assert st["preemptions"] > 0 and st["free_slots"] == 5 and st["free_pages"] == [-(-150 // bs)]
    eng.runner.ops.check_async_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefix_sharing_gives_the_same_tokens_with_fewer_positions_computed(tmp_path, dtype):
    """Requests whose prompts begin alike take over the full cache pages of the common prefix
    (several at once, one after another, and after the pages' first owner is gone); so few pages
    that registered pages are reclaimed in between.  The tokens are the plain implementation's."""
    name = "B"
    d = make_model_dir(tmp_path, name, dtype, std=GEN_STD[name])
    cfg, w = P.read_model_dir(d)
    V = cfg["vocab_size"]
    bs = TINY[name][1]
    stem_a, stem_b = random_prompt(V, 61, 400), random_prompt(V, 37, 401)
    prompts = [stem_a + random_prompt(V, n, 410 + i) for i, n in enumerate((3, 9, 1, 20))] + \
              [stem_b + random_prompt(V, n, 420 + i) for i, n in enumerate((5, 2))] + [stem_a[:40], stem_a + [7]]
    lens = [10, 6, 12, 5, 8, 9, 4, 6]

    def run(sharing, num_blocks):
        eng = Engine(str(d), dtype=dtype, block_size=bs, num_blocks=num_blocks, max_num_seqs=3, max_num_batched_tokens=40,
                     prefix_sharing=sharing)
        got, ids = {}, []
        pending = list(zip(prompts, lens))
        while pending or eng.has_unfinished():
            if pending and len(ids) - eng.stats()["finished"] < 3:
                p, n = pending.pop(0)
                ids.append(eng.add_request(p, SamplingParams.greedy(max_tokens=n)))
            for rid, tok, done in eng.step():
                got.setdefault(rid, []).append(tok)
        eng.runner.cache.check_integrity()
        return [got[i] for i in ids], eng.stats()

    want = [P.greedy_generate(cfg, w, p, n) for p, n in zip(prompts, lens)]

    def same(got):
        # float32: the plain implementation's tokens exactly.  bfloat16: every token the plain
        # argmax given the stream so far, or a near-tie of it
        if dtype == "float32":
            return got == want
        for g, p, n in zip(got, prompts, lens):
            check_greedy_stream(plain_forward(cfg, w), p, g, dtype, n, what="tiny B prefix sharing")
        return True

    out, st = run(True, 40)
    base, st0 = run(False, 40)
    assert same(out) and same(base)
    assert st0["prefix_hits"] == 0 and st["prefix_hits"] >= 3 * (61 // bs) * bs
    assert st["tokens_run"] < st0["tokens_run"] - st["prefix_hits"] // 2
    assert st["free_pages"] == [40]
    tight, st2 = run(True, 26)                       # registered pages have to make room
    assert same(tight) and st2["free_pages"] == [26]


@pytest.mark.parametrize("name", ["B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logits_over_adopted_pages(tmp_path, name, dtype):
    """The logits of a request that took over another request's pages -- a portion with a query
    offset over pages it did not write, then decoded tokens over them, also after the pages'
    first owner is gone and after a preempted request took them over again -- against the plain
    implementation and against the same steps without sharing."""
    d = make_model_dir(tmp_path, name, dtype)
    cfg, w = P.read_model_dir(d)
    V = cfg["vocab_size"]
    bs = TINY[name][1]
    stem = random_prompt(V, 5 * bs + 3, 500)
    first = stem + random_prompt(V, 9, 501)
    second = stem + random_prompt(V, 2 * bs + 1, 502)
    ref = P.forward_all_positions(cfg, w, second)
    scale = float(ref.abs().max())
    bound = 1e-4 if dtype == "float32" else bf16_bound(name) * scale

    def run(sharing):
        r = ModelRunner(d, engine_config=EngineConfig(dtype=dtype, block_size=bs, num_blocks=12 * 64 // bs, max_num_seqs=3,
                                                      max_num_batched_tokens=256, prefix_sharing=sharing))
        cm = r.cache
        s1 = r.admit()
        r.step([StepEntry(s1, first, ())])
        cm.register_prefix(s1, first, len(first))
        outs = []
        for round_ in range(2):                      # the second time the first owner is gone
            s2 = r.admit()
            n0 = cm.adopt_prefix(s2, second)
            # the stem's five full pages; the second time also the two this request registered itself
            assert n0 == ((5 if round_ == 0 else 7) * bs if sharing else 0)
            cut = max(n0 + 2, len(second) - 4)
            lg = r.step([StepEntry(s2, second[n0:cut], tuple(range(cut - n0)))]).float().cpu().clone()
            rows = [lg]
            for t in second[cut:]:
                r.decode_step([s2], [t], [0.0], [0])
                rows.append(r.last_logits[:1].float().cpu().clone())
            outs.append((n0, torch.cat(rows)))
            cm.register_prefix(s2, second, len(second))
            r.release(s2)
            if round_ == 0:
                r.release(s1)
            cm.check_integrity()
        r.ops.check_async_errors()
        return outs

    shared, alone = run(True), run(False)
    for (n0, got), (_, base) in zip(shared, alone):
        err = float((got - ref[n0:]).abs().max())
        if dtype != "float32":
            observe(f"tiny {name} logits over adopted pages", err, scale, bf16_bound(name))
        assert err <= bound, f"{err:.3e} > {bound:.3e}"
        # the same positions computed with pages of its own: the difference is what the kernels'
        # row counts make of rounding, nothing more
        assert float((got - base[n0:]).abs().max()) <= (0.0 if dtype == "float32" else bound)


def test_session_single_stream_calls(tmp_path):
    d = make_model_dir(tmp_path, "A", "float32")
    cfg, w = P.read_model_dir(d)
    toks = random_prompt(512, 30, 4)
    ref = P.forward_all_positions(cfg, w, toks)
    eng = Engine(str(d), dtype="float32", max_num_seqs=2)
    ses = Session(eng.runner, chunk=7)
    lg = ses.forward_logits(toks[:20])
    assert float((lg.cpu() - ref[19]).abs().max()) < 1e-4 and ses.position == 20
    t = ses.generate_token(toks[20:21])
    assert t == int(ref[20].argmax()) and ses.position == 21
    ses.truncate_to(12)                          # back to position 12, then the same tokens again
    assert ses.position == 12
    lg = ses.forward_logits(toks[12:21])
    assert float((lg.cpu() - ref[20]).abs().max()) < 1e-4 and ses.position == 21
    ses.reset_position()
    assert ses.position == 0
    allp = ses.forward_all_logits(toks)
    assert float((allp.cpu() - ref).abs().max()) < 1e-4
    ses.close()


def test_command_line(tmp_path):
    d = make_model_dir(tmp_path, "A", "float32", std=0.3)
    cfg, w = P.read_model_dir(d)
    prompt = random_prompt(512, 9, 8)
    want = P.greedy_generate(cfg, w, prompt, 6)
    cmd = [sys.executable, "-m", "zllm_b200", "generate", "--model", str(d), "--prompt-ids",
           ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0", "--dtype", "float32"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=str(TR.ROOT))
    assert p.returncode == 0, p.stderr[-2000:]
    assert " ".join(map(str, want)) in p.stdout and "--- 6 tokens in" in p.stdout
    # the random-weights mode from the command line
    (tmp_path / "c.json").write_text((d / "config.json").read_text())
    p = subprocess.run([sys.executable, "-m", "zllm_b200", "random", "--config", str(tmp_path / "c.json"), "--out",
                        str(tmp_path / "m2"), "--seed", "3"], capture_output=True, text=True, cwd=str(TR.ROOT))
    assert p.returncode == 0 and (tmp_path / "m2" / "model.safetensors").exists()
