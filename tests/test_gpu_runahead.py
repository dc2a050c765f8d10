"""The engine's run-ahead on the GPU: while only decoding, ``Engine.step`` launches the next
decode graph before it has read the tokens of the one in flight.  A request that ends on a stop
token, or is cancelled, meanwhile has one step too many computed and its slot is given back
while a graph that still names it may be in flight.  The reference tests the same schedules:
zllm src/backend/gpu/mod.rs:4105 (``gpu_cancel``) and :3554 (``gpu_continuous_batch``)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import plain_llama as P
from configs import GEN_STD, TINY, make_model_dir, random_prompt
from gpu_util import check_greedy_stream
from zllm_b200 import Engine, SamplingParams

def setup(tmp_path, name, dtype, slots=4):
    d = make_model_dir(tmp_path, name, dtype, std=GEN_STD[name])
    cfg, w = P.read_model_dir(d)
    bs = TINY[name][1]
    eng = Engine(str(d), dtype=dtype, block_size=bs, num_blocks=slots * (256 // bs), max_num_seqs=slots,
                 max_num_batched_tokens=128)
    assert eng.overlap and eng.runner.ecfg.cuda_graphs
    return eng, cfg, w, (lambda toks: P.forward_all_positions(cfg, w, toks))


def drain(eng, got, steps=None, ahead_seen=None):
    n = 0
    while eng.has_unfinished() and (steps is None or n < steps):
        for rid, tok, done in eng.step():
            got.setdefault(rid, []).append(tok)
        if ahead_seen is not None and eng._ahead is not None:
            ahead_seen.append(eng.steps)
        eng.runner.cache.check_integrity()
        n += 1


def all_free(eng, slots=4):
    st = eng.stats()
    eng.runner.cache.check_integrity()
    eng.runner.ops.check_async_errors()
    return st["free_slots"] == slots and st["free_pages"] == [eng.runner.cache.groups[0].pool.num_pages] \
        and st["running"] == 0 and st["prefilling"] == 0 and st["waiting"] == 0


@pytest.mark.parametrize("name", ["C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_stop_token_ends_one_of_four_requests_while_a_step_is_in_flight(tmp_path, name, dtype):
    eng, cfg, w, fwd = setup(tmp_path, name, dtype)
    V = cfg["vocab_size"]
    prompts = [random_prompt(V, n, 600 + n) for n in (7, 19, 4, 40)]
    N = 24
    # the engine's own streams without a stop token (checked against plain), to pick the stop from
    free_run = eng.generate(prompts, SamplingParams.greedy(max_tokens=N))
    for p, o in zip(prompts, free_run):
        check_greedy_stream(fwd, p, o, dtype, N, what=f"tiny {name} run-ahead")
    if dtype == "float32":
        assert free_run == [P.greedy_generate(cfg, w, p, N) for p in prompts]
    # a token of request 1's stream that appears first at a step in the middle, not the last
    k = next(i for i in range(6, N - 4) if free_run[1][i] not in free_run[1][:i])
    stop = free_run[1][k]
    params = [SamplingParams.greedy(max_tokens=N) for _ in prompts]
    params[1] = SamplingParams(temperature=0.0, max_tokens=N, stop_token_ids=(stop,))
    ids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
    got, ahead = {}, []
    drain(eng, got, ahead_seen=ahead)
    assert ahead, "the engine never ran ahead: the test did not exercise what it is for"
    assert got[ids[1]] == free_run[1][:k + 1]            # the stop token is emitted, nothing after it
    for i in (0, 2, 3):                                   # the others do not notice
        check_greedy_stream(fwd, prompts[i], got[ids[i]], dtype, N, what=f"tiny {name} run-ahead")
        if dtype == "float32":
            assert got[ids[i]] == free_run[i]
    assert eng.scheduler.requests[ids[1]].finish_reason == "stop"
    assert all_free(eng)


@pytest.mark.parametrize("name", ["C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cancel_between_steps_then_a_new_request_in_the_freed_slot(tmp_path, name, dtype):
    eng, cfg, w, fwd = setup(tmp_path, name, dtype)
    V = cfg["vocab_size"]
    prompts = [random_prompt(V, n, 700 + n) for n in (9, 3, 30, 14)]
    N = 20
    ids = [eng.add_request(p, SamplingParams.greedy(max_tokens=N)) for p in prompts]
    got = {}
    drain(eng, got, steps=8)
    assert eng._ahead is not None                          # a decode step is in flight right now
    victim = ids[2]
    slot = eng.scheduler.requests[victim].slot
    produced = len(got[victim])
    assert eng.cancel(victim) and not eng.cancel(victim)
    eng.runner.cache.check_integrity()
    # a new request arrives at once; it gets the freed slot
    newcomer = random_prompt(V, 11, 777)
    nid = eng.add_request(newcomer, SamplingParams.greedy(max_tokens=N))
    drain(eng, got)
    assert eng.scheduler.requests[nid].finish_reason == "length"
    assert len(got[victim]) == produced                    # nothing was reported for it after the cancel
    for i, p in zip(ids, prompts):
        if i != victim:
            check_greedy_stream(fwd, p, got[i], dtype, N, what=f"tiny {name} cancel")
    check_greedy_stream(fwd, prompts[2], got[victim], dtype, produced, what=f"tiny {name} cancel")
    check_greedy_stream(fwd, newcomer, got[nid], dtype, N, what=f"tiny {name} cancel")
    if dtype == "float32":
        assert got[nid] == P.greedy_generate(cfg, w, newcomer, N)
    assert slot is not None and all_free(eng)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_stops_while_another_is_admitted(tmp_path, dtype):
    """The step in which a request ends by its stop token is also the step before a waiting
    request gets its slot: the run-ahead must give way to a scheduled step."""
    name = "C"
    eng, cfg, w, fwd = setup(tmp_path, name, dtype, slots=2)
    V = cfg["vocab_size"]
    prompts = [random_prompt(V, n, 800 + n) for n in (6, 12, 21)]
    N = 18
    free_run = eng.generate(prompts[:2], SamplingParams.greedy(max_tokens=N))
    k = next(i for i in range(5, N - 3) if free_run[0][i] not in free_run[0][:i])
    params = [SamplingParams(temperature=0.0, max_tokens=N, stop_token_ids=(free_run[0][k],)),
              SamplingParams.greedy(max_tokens=N), SamplingParams.greedy(max_tokens=N)]
    ids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]      # two slots: the third waits
    got = {}
    drain(eng, got)
    assert got[ids[0]] == free_run[0][:k + 1]
    for i in (1, 2):
        check_greedy_stream(fwd, prompts[i], got[ids[i]], dtype, N, what=f"tiny {name} stop and admit")
    if dtype == "float32":
        assert got[ids[2]] == P.greedy_generate(cfg, w, prompts[2], N)
    assert all_free(eng, slots=2)
