"""The engine's host side on the CPU: cache, tables, batch description, step function and
scheduler run the four ways of cutting with the plain torch statements of the kernels
(``ref_ops``) in place of the CUDA kernels, and must reproduce the plain whole-sequence
implementation.  (The product has no CPU path; the kernels' own tests are GPU tests.)"""
import pytest
import torch

import plain_llama as P
import traces as TR
from configs import TINY, make_model_dir, random_prompt
from ref_ops import RefOps
from zllm_b200 import Engine, EngineConfig, ModelRunner, SamplingParams
from zllm_b200.errors import MemoryError_, RequestError
from zllm_b200 import StepEntry


def cpu_runner(model_dir, name, num_blocks, max_rows=256, slots=8):
    return ModelRunner(model_dir, ops=RefOps(), engine_config=EngineConfig(
        dtype="float32", device="cpu", cuda_graphs=False, block_size=TINY[name][1], num_blocks=num_blocks,
        max_num_seqs=slots, max_num_batched_tokens=max_rows))


@pytest.mark.parametrize("name", ["A", "B"])
def test_four_ways_of_cutting_agree_with_plain(tmp_path, name):
    d = make_model_dir(tmp_path, name)
    cfg, w = P.read_model_dir(d)
    V = cfg["vocab_size"]
    reqs = [(f"r{i}", random_prompt(V, n, 10 + i)) for i, n in enumerate((5, 49, 33, 70, 17, 64))]
    ref = {rid: P.forward_all_positions(cfg, w, toks) for rid, toks in reqs}
    max_tokens = 256
    steps = (TR.family_whole(reqs, "w.") + TR.family_tail(reqs, 32, "t.") + TR.family_portions(reqs, prefix="p.")
             + TR.family_mixed(reqs, max_tokens, 4, 1, "m."))
    assert TR.live_tokens_needed(steps) <= max_tokens
    runner = cpu_runner(d, name, max_tokens // TINY[name][1])
    got = TR.replay_inprocess(runner, steps)
    for prefix in ("w.", "t.", "p.", "m."):
        TR.compare(got, ref, reqs, prefix, 2e-5, 0.0, f"tiny {name} {prefix}")
    assert runner.cache.free_pages() == [max_tokens // TINY[name][1]]


def test_step_errors_are_raised_before_anything_runs(tmp_path):
    d = make_model_dir(tmp_path, "A")
    r = cpu_runner(d, "A", num_blocks=4, max_rows=64)
    s = r.admit()
    with pytest.raises(RequestError, match="at least one token"):
        r.step([StepEntry(s, [], ())])
    with pytest.raises(RequestError, match="twice"):
        r.step([StepEntry(s, [1], ()), StepEntry(s, [2], ())])
    with pytest.raises(RequestError, match="max_num_batched_tokens"):
        r.step([StepEntry(s, [1] * 65, ())])
    s2 = r.admit()
    r.step([StepEntry(s, [1] * 40, ())])
    free = r.cache.free_pages()
    with pytest.raises(MemoryError_, match="exhausted"):
        r.step([StepEntry(s2, [1] * 30, ())])
    assert r.cache.free_pages() == free and r.cached_len(s2) == 0     # nothing was taken or run
    r.cache.check_integrity()
    with pytest.raises(RequestError, match="not live"):
        r.step([StepEntry(5, [1], ())])


def test_generation_is_unchanged_by_preemption_and_portions(tmp_path):
    d = make_model_dir(tmp_path, "A", std=0.3)
    cfg, w = P.read_model_dir(d)
    prompts = [random_prompt(512, n, 20 + n) for n in (5, 17, 33, 15)]
    want = [P.greedy_generate(cfg, w, p, 24) for p in prompts]
    for nb, budget, slots in ((64, 256, 4), (8, 16, 3), (7, 9, 4)):
        eng = Engine(str(d), ops=RefOps(), dtype="float32", device="cpu", cuda_graphs=False, block_size=16,
                     num_blocks=nb, max_num_seqs=slots, max_num_batched_tokens=budget)
        out = eng.generate(prompts, SamplingParams.greedy(max_tokens=24))
        assert out == want, f"pool {nb}, budget {budget}"
        st = eng.stats()
        assert st["free_pages"] == [nb] and st["free_slots"] == slots
        if nb == 7:
            assert st["preemptions"] > 0
        eng.runner.cache.check_integrity()


def test_temperature_sampling_is_reproducible_and_survives_preemption(tmp_path):
    d = make_model_dir(tmp_path, "B", std=0.2)
    prompts = [random_prompt(1000, n, 40 + n) for n in (3, 30, 12)]
    params = [SamplingParams.with_temperature(0.8, seed=100 + i, max_tokens=20) for i in range(3)]

    def run(nb, budget):
        eng = Engine(str(d), ops=RefOps(), dtype="float32", device="cpu", cuda_graphs=False, block_size=8,
                     num_blocks=nb, max_num_seqs=3, max_num_batched_tokens=budget)
        out = eng.generate(prompts, params)
        return out, eng.stats()["preemptions"]

    a, _ = run(64, 64)
    b, pre = run(12, 13)
    assert a == b and pre > 0
    greedy, _ = run(64, 64) if False else (None, None)
    cfg, w = P.read_model_dir(d)
    # token n of a request is the Gumbel-max draw with seed base + n * 0x9E3779B1 on the plain logits
    toks = list(prompts[0])
    for n in range(3):
        lg = P.forward_all_positions(cfg, w, toks)[-1]
        t = P.gumbel_sample(lg, 0.8, P.step_seed(100, n))
        assert t == a[0][n]
        toks.append(t)


def test_workspace_keeps_a_buffer_that_had_to_grow():
    """Captured graphs hold the addresses of the buffers they were captured with: a buffer that is
    replaced by a larger one must stay allocated."""
    import torch
    from zllm_b200.engine.batch import Workspace
    ws = Workspace(16, "cpu")
    a = ws.get("partials", (2, 8), torch.float32, cap=2)
    a.fill_(3.0)
    old = a.data_ptr()
    del a
    b = ws.get("partials", (5, 8), torch.float32, cap=5)
    assert b.shape == (5, 8) and b.data_ptr() != old
    assert any(t.data_ptr() == old and float(t.sum()) == 48.0 for t in ws._retired)
    assert ws.get("partials", (3, 8), torch.float32, cap=3).data_ptr() == b.data_ptr()
    assert ws.bytes() == (2 + 5) * 8 * 4


def test_prefix_sharing_and_truncation_leave_the_tokens_unchanged(tmp_path):
    """The engine with the reference kernels on the CPU: requests with common prefixes take over
    each other's pages (also after a preemption, and with pages reclaimed in between); a
    session goes back and forth with ``truncate_to``.  Every token is the plain implementation's."""
    from zllm_b200 import Session
    d = make_model_dir(tmp_path, "A", "float32", std=0.3)
    cfg, w = P.read_model_dir(d)
    stem = random_prompt(512, 45, 60)
    prompts = [stem + random_prompt(512, n, 61 + n) for n in (4, 11, 2)] + [stem[:30], random_prompt(512, 20, 70)]
    want = [P.greedy_generate(cfg, w, p, 7) for p in prompts]
    for nb, budget in ((40, 64), (10, 9)):
        ecfg = EngineConfig(dtype="float32", device="cpu", block_size=16 if nb == 40 else 8, num_blocks=nb, max_num_seqs=3,
                            max_num_batched_tokens=budget, cuda_graphs=False, prefix_sharing=True)
        eng = Engine(str(d), ops=RefOps(), engine_config=ecfg)
        assert eng.generate(prompts, SamplingParams.greedy(max_tokens=7)) == want
        st = eng.stats()
        eng.runner.cache.check_integrity()
        assert st["prefix_hits"] > 0 and st["free_pages"] == [nb]
        assert eng.generate(prompts[:2], SamplingParams.greedy(max_tokens=7)) == want[:2]   # found again later
    assert st["preemptions"] > 0
    ses = Session(eng.runner, chunk=5)
    toks = prompts[1]
    ref = P.forward_all_positions(cfg, w, toks)
    ses.forward_logits(toks[:33])
    for back in (32, 17, 0, 8):                      # 17 lies inside a page that other requests registered
        try:
            ses.truncate_to(back)
        except MemoryError_:
            ses.truncate_to(back - back % 8)
        lg = ses.forward_logits(toks[ses.position:40])
        assert float((lg - ref[39]).abs().max()) < 1e-4
    ses.close()
    eng.runner.cache.check_integrity()


def test_a_kernels_error_flag_stops_the_engine(tmp_path):
    """The engine asks the kernel table for flagged bounded waits where it has just synchronised
    (after the sampler's copy, after collecting a decode step); a table that reports one makes the
    step raise instead of handing out tokens computed from an abandoned launch."""
    from zllm_b200.errors import BackendError

    class FlaggingOps(RefOps):
        flagged = False

        def raise_if_a_wait_gave_up(self):
            if self.flagged:
                raise BackendError("gemm_tc: a bounded wait ran out (code 3); results of that launch are invalid")

    d = make_model_dir(tmp_path, "A")
    ops = FlaggingOps()
    eng = Engine(str(d), ops=ops, dtype="float32", device="cpu", cuda_graphs=False, block_size=16, num_blocks=16,
                 max_num_seqs=2, max_num_batched_tokens=32)
    eng.add_request(random_prompt(512, 9, 1), SamplingParams.greedy(max_tokens=4))
    assert len(eng.step()) == 1                       # the prompt's step: one token
    ops.flagged = True
    with pytest.raises(BackendError, match="bounded wait ran out"):
        eng.step()
