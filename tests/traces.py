"""Traces: the same requests cut into steps in different ways, in the format that
``bin/trace_run`` reads, and two ways to replay them (in-process and through the program).

A request is (id, tokens): prompt and teacher-forced continuation alike are just
tokens, so every way of cutting sees identical inputs.  Every position's logits are
wanted; results are keyed by (request, position).
"""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def _entry(rid, tokens, start, n):
    return {"id": rid, "tokens": tokens[start:start + n], "want": list(range(n))}


def family_whole(reqs, prefix=""):
    """Each request alone and whole: one step per request."""
    steps = []
    for rid, toks in reqs:
        steps.append({"entries": [_entry(prefix + rid, toks, 0, len(toks))], "end": [prefix + rid]})
    return steps


def family_tail(reqs, tail=32, prefix=""):
    """Most of it in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in reqs:
        head = max(1, len(toks) - tail)
        steps.append({"entries": [_entry(prefix + rid, toks, 0, head)], "end": []})
        for p in range(head, len(toks)):
            steps.append({"entries": [_entry(prefix + rid, toks, p, 1)], "end": [prefix + rid] if p == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [prefix + rid]
    return steps


def family_portions(reqs, sizes=(7, 13, 2, 64, 1, 3, 2, 31, 5, 2, 16, 1, 1, 40), prefix=""):
    """Portions of changing size, down to two tokens (and single ones)."""
    steps = []
    for k, (rid, toks) in enumerate(reqs):
        p, i = 0, k            # each request starts at another place of the size list
        while p < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - p)
            i += 1
            steps.append({"entries": [_entry(prefix + rid, toks, p, n)], "end": [prefix + rid] if p + n == len(toks) else []})
            p += n
    return steps


def family_mixed(reqs, max_tokens, max_live=4, seed=0, prefix=""):
    """Up to ``max_live`` live requests; portions of some beside single tokens of others; a
    request may sit out a step; a new one starts when the rounded-up sizes of the live ones
    leave room in ``max_tokens`` -- so finished requests' pages are handed to later ones."""
    rng = random.Random(seed)
    pending = list(reqs)
    live = {}           # rid -> [tokens, position, mode]
    steps = []
    up = lambda n: -(-n // 64) * 64
    while pending or live:
        while pending and len(live) < max_live and \
                sum(up(len(v[0])) for v in live.values()) + up(len(pending[0][1])) <= max_tokens:
            rid, toks = pending.pop(0)
            live[prefix + rid] = [toks, 0, rng.choice(["portions", "tail"])]
        entries, end = [], []
        for rid in list(live):
            toks, p, mode = live[rid]
            if len(live) > 1 and rng.random() < 0.15:
                continue                                   # left out of this step, goes on later
            left = len(toks) - p
            if mode == "tail" and left > 20:
                n = left - 20 if p == 0 else 1
            elif mode == "tail":
                n = 1
            else:
                n = rng.choice([1, 1, 2, 2, 3, 7, 16, 33])
            n = max(1, min(n, left))
            entries.append(_entry(rid, toks, p, n))
            live[rid][1] = p + n
            if p + n == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def number(steps, first=0):
    return [dict(s, step=first + i) for i, s in enumerate(steps)]


def live_tokens_needed(steps):
    """The most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held, worst = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // 64) * 64 for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


# ---------------------------------------------------------------------------------------
def replay_inprocess(runner, steps):
    """Drive a ModelRunner directly; returns {(id, position): logits row (CPU float32)}."""
    from zllm_b200 import StepEntry
    slots, pos, out = {}, {}, {}
    for s in steps:
        ents = []
        for e in s["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = runner.admit()
                assert slots[e["id"]] is not None, "no free slot"
                pos[e["id"]] = 0
            ents.append(StepEntry(slots[e["id"]], e["tokens"], tuple(e["want"])))
        logits = runner.step(ents)
        if logits is not None:
            logits = logits.detach().float().cpu()
            r = 0
            for e in s["entries"]:
                for w in e["want"]:
                    out[(e["id"], pos[e["id"]] + w)] = logits[r].clone()
                    r += 1
        for e in s["entries"]:
            pos[e["id"]] += len(e["tokens"])
        for rid in s["end"]:
            runner.release(slots.pop(rid))
        runner.cache.check_integrity()
    return out


def replay_program(model_dir, dtype, steps, max_tokens, out_dir, vocab, extra_args=(), env=None):
    """Run ``bin/trace_run`` on the steps; returns {(id, position): logits row}."""
    steps = number(steps)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra_args]
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=900, env=env)
    assert proc.returncode == 0, f"trace_run exit {proc.returncode}\nstdout:\n{proc.stdout[-2000:]}\nstderr:\n{proc.stderr[-4000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    pos, out = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        f = Path(out_dir) / f"{s['step']}.f32"
        if n_want == 0:
            assert not f.exists()
        else:
            arr = np.fromfile(f, dtype="<f4")
            assert arr.size == n_want * vocab, f"{f}: {arr.size} values, expected {n_want}x{vocab}"
            arr = torch.from_numpy(arr.reshape(n_want, vocab).copy())
            r = 0
            for e in s["entries"]:
                for w in e["want"]:
                    out[(e["id"], pos.get(e["id"], 0) + w)] = arr[r]
                    r += 1
        for e in s["entries"]:
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
    return out


def compare(got, reference, reqs, prefix, atol, rtol_of_scale, what):
    """Every (request, position) of ``got`` against the plain logits ``reference[rid][pos]``.
    The worst error, as a fraction of the request's largest |logit|, is recorded under ``what``."""
    from gpu_util import observe
    worst, worst_at = 0.0, None
    for rid, toks in reqs:
        ref = reference[rid]
        scale = float(ref.abs().max())
        for p in range(len(toks)):
            row = got.get((prefix + rid, p))
            assert row is not None, f"{what}: no logits for request {rid} position {p}"
            err = float((row - ref[p]).abs().max())
            bound = atol + rtol_of_scale * scale
            if err > worst:
                worst, worst_at = err, (rid, p)
            if rtol_of_scale > 0:
                observe(what, err, scale, rtol_of_scale)
            assert err <= bound, (f"{what}: request {rid} position {p} (first wrong place): "
                                  f"max abs error {err:.3e} > {bound:.3e}")
    return worst, worst_at
