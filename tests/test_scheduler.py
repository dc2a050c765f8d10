"""The scheduler's decisions (CPU): admission, portions under the token budget, decoding,
finishing and freeing, and what happens when pages run out.  A stand-in executor does what
the step function does to the cache (ensure, advance) and returns deterministic tokens."""
import pytest
import torch

from zllm_b200.cache import CacheManager
from zllm_b200.engine.scheduler import FINISHED, PREEMPTED, Scheduler
from zllm_b200.errors import RequestError
from zllm_b200.parts import KVCacheSpec
from zllm_b200.sampling import SamplingParams


def make(n_pages=32, bs=4, slots=4, budget=16, max_len=64):
    cm = CacheManager([(KVCacheSpec(1, 16), None)], bs, n_pages, slots, max_len, torch.float32, "cpu", allocate=False)
    return cm, Scheduler(cm, budget, max_len)


def token_for(req, position):
    return (req.id * 1000 + position * 7) % 997          # depends only on (request, position)


def run_step(cm, sch, log=None):
    plan = sch.schedule()
    if plan.empty:
        return plan, []
    assert plan.num_tokens <= sch.budget
    for r in plan.decodes:
        assert cm.ensure(r.slot, len(r.tokens))
        cm.advance(r.slot, len(r.tokens))
    for p in plan.portions:
        assert cm.length[p.request.slot] == p.start
        assert cm.ensure(p.request.slot, p.start + p.n)
        cm.advance(p.request.slot, p.start + p.n)
    dec = [token_for(r, len(r.tokens)) for r in plan.decodes]
    first = [token_for(p.request, len(p.request.tokens)) if p.completes else None for p in plan.portions]
    out = sch.commit(plan, dec, first)
    cm.check_integrity()
    if log is not None:
        log.append((plan, out))
    return plan, out


def drain(cm, sch, limit=2000):
    outs = {}
    for _ in range(limit):
        if not sch.has_unfinished():
            break
        _, out = run_step(cm, sch)
        for rid, tok, done in out:
            outs.setdefault(rid, []).append(tok)
    assert not sch.has_unfinished()
    return outs


def test_rejections():
    cm, sch = make(n_pages=4, max_len=32)
    with pytest.raises(RequestError, match="empty"):
        sch.add([], SamplingParams.greedy())
    with pytest.raises(RequestError, match="maximum length"):
        sch.add(list(range(32)), SamplingParams.greedy())
    with pytest.raises(RequestError, match="never fit"):
        sch.add(list(range(10)), SamplingParams.greedy(max_tokens=20))     # 30 positions > 4 pages of 4
    with pytest.raises(RequestError, match="max_tokens"):
        sch.add([1], SamplingParams(max_tokens=0))


def test_prompt_is_cut_into_portions_under_the_budget_and_first_token_comes_with_the_last():
    cm, sch = make(budget=16)
    rid = sch.add(list(range(40)), SamplingParams.greedy(max_tokens=3))
    sizes, produced = [], []
    while sch.has_unfinished():
        plan, out = run_step(cm, sch)
        sizes.append([(p.start, p.n, p.completes) for p in plan.portions])
        produced.append(out)
    assert sizes[:3] == [[(0, 16, False)], [(16, 16, False)], [(32, 8, True)]]
    assert produced[0] == [] and produced[1] == [] and len(produced[2]) == 1
    assert [o[0][2] for o in produced[2:]] == [False, False, True]
    assert sch.requests[rid].state == FINISHED and sch.requests[rid].finish_reason == "length"
    assert cm.free_pages() == [32] and len(cm.free_slots) == 4


def test_decodes_go_first_and_portions_of_several_requests_share_one_step():
    cm, sch = make(budget=16)
    a = sch.add(list(range(6)), SamplingParams.greedy(max_tokens=10))
    run_step(cm, sch)                                # a prefilled whole, now running
    b = sch.add(list(range(9)), SamplingParams.greedy(max_tokens=10))
    c = sch.add(list(range(30)), SamplingParams.greedy(max_tokens=10))
    plan, out = run_step(cm, sch)
    assert [r.id for r in plan.decodes] == [a]
    assert [(p.request.id, p.n, p.completes) for p in plan.portions] == [(b, 9, True), (c, 6, False)]
    assert plan.num_tokens == 16
    assert [o[0] for o in out] == [a, b]
    plan, _ = run_step(cm, sch)
    assert [r.id for r in plan.decodes] == [a, b] and [(p.request.id, p.start, p.n) for p in plan.portions] == [(c, 6, 14)]


def test_stop_token_is_emitted_and_frees_at_once():
    cm, sch = make()
    rid = sch.add([1, 2, 3], SamplingParams.greedy(max_tokens=50))
    r = sch.requests[rid]
    stop = token_for(r, 5)                            # the token produced when 5 tokens are held
    r.params.stop_token_ids = (stop,)
    outs = drain(cm, sch)
    assert outs[rid][-1] == stop and len(outs[rid]) == 3 and r.finish_reason == "stop"
    assert cm.free_pages() == [32]


def test_waiting_requests_get_slots_in_order():
    cm, sch = make(slots=2, budget=64)
    ids = [sch.add(list(range(5)), SamplingParams.greedy(max_tokens=2 + i)) for i in range(5)]
    firsts = []
    for _ in range(40):
        if not sch.has_unfinished():
            break
        plan, _ = run_step(cm, sch)
        firsts += [p.request.id for p in plan.portions if p.start == 0]
        assert len(sch.running) + len(sch.prefilling) <= 2
    assert firsts == ids and sch.finished == 5


def test_when_pages_run_out_the_newest_running_request_is_preempted_and_resumed():
    # 3 requests of 3 tokens (1 page each) growing to 19 tokens (5 pages each) in a pool of 8 pages
    cm, sch = make(n_pages=8, bs=4, slots=3, budget=32, max_len=32)
    ids = [sch.add([i, i + 1, i + 2], SamplingParams.greedy(max_tokens=16)) for i in range(3)]
    log = []
    outs = {}
    for _ in range(400):
        if not sch.has_unfinished():
            break
        _, out = run_step(cm, sch, log)
        for rid, tok, done in out:
            outs.setdefault(rid, []).append(tok)
    assert sch.preemptions > 0 and sch.finished == 3
    # the victim of the first preemption is the most recently admitted running request
    first_victim = next(r for r in sch.requests.values() if r.id == ids[2])
    assert first_victim.finish_reason == "length"
    # every request produced exactly the tokens it would have produced alone
    for rid in ids:
        r = sch.requests[rid]
        assert outs[rid] == [token_for(r, 3 + k) for k in range(16)]
    assert cm.free_pages() == [8] and len(cm.free_slots) == 3


def test_the_last_running_request_is_never_preempted():
    cm, sch = make(n_pages=6, bs=4, slots=2, budget=8, max_len=24)
    a = sch.add([1, 2, 3], SamplingParams.greedy(max_tokens=20))
    b = sch.add([4, 5, 6], SamplingParams.greedy(max_tokens=20))
    seen_alone = False
    for _ in range(200):
        if not sch.has_unfinished():
            break
        run_step(cm, sch)
        if sch.requests[b].state == PREEMPTED:
            seen_alone = True
            assert sch.requests[a].state in ("running", FINISHED)
    assert seen_alone and sch.finished == 2


def test_front_prefill_has_priority_over_running_requests():
    cm, sch = make(n_pages=8, bs=4, slots=3, budget=64, max_len=32)
    a = sch.add(list(range(10)), SamplingParams.greedy(max_tokens=20))
    run_step(cm, sch)                                  # a running, holds 3 pages
    for _ in range(5):
        run_step(cm, sch)                              # a grows to 16 positions: 4 pages
    b = sch.add(list(range(14)), SamplingParams.greedy(max_tokens=4))   # 4 pages: admitted (fits now)
    plan, _ = run_step(cm, sch)
    assert any(p.request.id == b for p in plan.portions)
    outs = drain(cm, sch)
    assert sch.finished == 2 and cm.free_pages() == [8]


def test_cancel_frees_wherever_the_request_is():
    cm, sch = make(slots=2, budget=8)
    a = sch.add(list(range(20)), SamplingParams.greedy(max_tokens=5))
    b = sch.add(list(range(5)), SamplingParams.greedy(max_tokens=5))
    c = sch.add(list(range(5)), SamplingParams.greedy(max_tokens=5))
    run_step(cm, sch)
    assert sch.cancel(c) and sch.cancel(a)             # waiting; prefilling
    assert not sch.cancel(a) and not sch.cancel(12345)
    outs = drain(cm, sch)
    assert list(outs) == [b] and len(outs[b]) == 5
    assert cm.free_pages() == [32] and len(cm.free_slots) == 2


@pytest.mark.parametrize("sharing", [False, True])
def test_random_workloads_keep_every_page_accounted(sharing, seed=3):
    import random
    rng = random.Random(seed)
    cm = CacheManager([(KVCacheSpec(1, 16), None)], 4, 20, 4, 40, torch.float32, "cpu", allocate=False,
                      prefix_sharing=sharing)
    sch = Scheduler(cm, 12, 40)
    stems = [[rng.randrange(500) for _ in range(20)] for _ in range(2)]
    expect = {}
    outs = {}
    pending = 25
    for step in range(3000):
        if pending and rng.random() < 0.3:
            n = rng.randint(1, 20)
            mt = rng.randint(1, 15)
            cut = rng.randint(0, n)                              # prompts begin with a piece of a common stem
            prompt = rng.choice(stems)[:cut] + [rng.randrange(500) for _ in range(n - cut)]
            rid = sch.add(prompt, SamplingParams.greedy(max_tokens=mt))
            expect[rid] = (n, mt)
            pending -= 1
        if rng.random() < 0.02 and sch.running:
            victim = rng.choice(sch.running).id
            sch.cancel(victim)
            expect.pop(victim)
        _, out = run_step(cm, sch)
        for rid, tok, done in out:
            outs.setdefault(rid, []).append(tok)
        if not pending and not sch.has_unfinished():
            break
    assert not sch.has_unfinished()
    for rid, (n, mt) in expect.items():
        r = sch.requests[rid]
        assert outs[rid] == [token_for(r, n + k) for k in range(min(mt, 40 - n))]
    assert cm.free_pages() == [20] and len(cm.free_slots) == 4
    assert (cm.prefix_hits > 0) == sharing


def test_a_request_with_a_known_prefix_starts_behind_it():
    cm = CacheManager([(KVCacheSpec(1, 16), None)], 4, 32, 4, 64, torch.float32, "cpu", allocate=False,
                      prefix_sharing=True)
    sch = Scheduler(cm, 16, 64)
    stem = list(range(200, 222))                             # 22 tokens: 5 full pages of 4
    a = sch.add(stem, SamplingParams.greedy(max_tokens=3))
    drain(cm, sch)
    assert sch.requests[a].state == FINISHED and cm.prefix_hits == 0
    assert cm.free_pages() == [32]                           # everything is free or waits to be found
    log = []
    b = sch.add(stem[:18] + [5, 6, 7], SamplingParams.greedy(max_tokens=2))
    run_step(cm, sch, log)
    plan, _ = log[0]
    assert [(p.request.id, p.start, p.n, p.completes) for p in plan.portions] == [(b, 16, 5, True)]
    assert cm.prefix_hits == 16 and sch.stats()["prefix_hits"] == 16
    drain(cm, sch)
    # a preempted request finds its own pages again when it is resumed
    c = sch.add(list(range(300, 330)), SamplingParams.greedy(max_tokens=4))
    run_step(cm, sch)
    run_step(cm, sch)
    rc = sch.requests[c]
    assert rc.num_computed == 30
    sch._preempt(sch.running.pop())
    log = []
    run_step(cm, sch, log)
    plan, _ = log[0]
    assert plan.portions[0].start == 28 and plan.portions[0].request.id == c      # 7 full pages taken over
    drain(cm, sch)
    assert cm.free_pages() == [32]
