#!/usr/bin/env python3
"""Benchmark: decoded tokens per second of the Llama-3.2-1B-shaped model (random weights,
bfloat16) on one B200, with prefill throughput, roofline fractions and end-to-end numbers.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]
    python bench.py --config 8b          # Llama-3.1-8B shape: decode to context 8192, prefill 2,048
    python bench.py --config 3b-mixed    # Llama-3.2-3B shape: 32 requests, 512-token portions beside decoding
    python bench.py --config cpu-baseline  # the plain CPU implementation of the test-suite, timed (no GPU)

One JSON line on stdout.  ``value``: decode tokens/s at batch 8 near context 4096, K decode
steps timed on the device with CUDA events (the steps replay a captured graph back to back,
each step's sampled token feeding the next).  ``e2e``: the same through ``Engine.step()``,
host tokens in (pinned buffer, one copy per step) and host tokens out.  ``prefill``: one
2,048-token prompt in one step.  ``roofline``: bytes a decode step must read (every weight
once + the cache of the live requests) / its time, against the measured HBM copy bandwidth.
``points``: decode tokens/s at batch 1 and 64.  The engine runs on one GPU: for N > 1 a line
says so and the exit code is 2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Llama-3.2-1B shape: the configuration the headline numbers are quoted on
MODEL = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=16, hidden_size=2048, num_attention_heads=32,
             num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256, rms_norm_eps=1e-5,
             rope_theta=500000.0,
             rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                               original_max_position_embeddings=8192),
             max_position_embeddings=131072, tie_word_embeddings=True)
# layer sizes of the larger Llama shapes, for --case runs at other sizes (--shape)
SHAPES = {
    "1b": {},
    "3b": dict(num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8, head_dim=128,
               intermediate_size=8192),
    "8b": dict(num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=14336, tie_word_embeddings=False,
               rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=8192)),
}
CONTEXT = 4096
PROMPT = 2048
BLOCK = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(d.get(k), (int, float)):
                out[k] = float(d[k])
        return out, "measured"
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        mhz, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                mhz.append(int(float(r[0])))
                mx = max(mx, int(float(r[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz)}


def model_numbers(cfg):
    """Bytes of weights a decode step reads, KV bytes per cached token, flops of a prefill."""
    H, I, V, L = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    nq, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_layer = (nq + 2 * nkv) * hd * H + H * nq * hd + 3 * I * H + 2 * H
    weight_bytes = 2 * (L * per_layer + V * H + H)          # bf16; the head reads the (tied) table once
    kv_per_token = 2 * L * nkv * hd * 2

    def prefill_flops(T):
        gemm = 2 * T * L * ((nq + 2 * nkv) * hd * H + H * nq * hd + 3 * I * H) + 2 * V * H
        attn = L * 4 * nq * hd * (T * (T + 1) // 2)          # causal QK^T and PV
        return gemm + attn
    return weight_bytes, kv_per_token, prefill_flops


def profile_case(args):
    """A small case for ncu: the same model shape (optionally fewer layers), graphs off so that
    every kernel is its own launch."""
    import torch
    from zllm_b200 import EngineConfig, LlamaConfig, ModelRunner, StepEntry

    shape = dict(MODEL, **SHAPES[args.shape])
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    cfg = LlamaConfig.from_dict(shape)
    pk, _ = peaks()
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg)
    B = args.batch
    ctx_len = args.context
    runner = ModelRunner(config=cfg, seed=2, random_on_device=True, engine_config=EngineConfig(
        dtype="bfloat16", block_size=BLOCK, num_blocks=B * (-(-(ctx_len + 64) // BLOCK)) + args.tokens // BLOCK + 8,
        max_num_seqs=max(B, 1), max_num_batched_tokens=max(args.tokens, PROMPT), max_model_len=max(ctx_len + 64, args.tokens + 8),
        cuda_graphs=bool(args.graphs)))
    gen = torch.Generator().manual_seed(0)
    rand = lambda n: torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.case == "prefill":
        toks = rand(args.tokens)
        times, wall = [], []
        for _ in range(max(2, args.steps)):
            s = runner.admit()
            torch.cuda.synchronize(); t0 = time.perf_counter(); a.record()
            runner.step([StepEntry(s, toks, (len(toks) - 1,))])
            b.record(); t1 = time.perf_counter(); torch.cuda.synchronize()
            times.append(round(a.elapsed_time(b), 4))
            wall.append(round((t1 - t0) * 1e3, 4))          # the host's share: until the last launch is issued
            runner.release(s)
        best = min(times)
        if runner.ops.profiling:                              # ZLLM_PROFILE=1: device time per kind of operation
            runner.ops.take_profile()
            s = runner.admit()
            runner.step([StepEntry(s, toks, (len(toks) - 1,))])
            print(json.dumps({"case": "prefill", "tokens": args.tokens, "kernel_ms": runner.ops.take_profile()}))
            runner.release(s)
        print(json.dumps({"case": "prefill", "shape": args.shape, "tokens": args.tokens, "layers": cfg.num_hidden_layers,
                          "graphs": bool(args.graphs), "ms": times, "host_ms": wall,
                          "tflops": round(prefill_flops(args.tokens) / best / 1e9, 1),
                          "frac_of_peak": round(prefill_flops(args.tokens) / best / 1e9 / pk["bf16_tflops"], 3)}))
        return 0
    slots = [runner.admit() for _ in range(B)]
    for s in slots:
        toks = rand(ctx_len)
        for i in range(0, ctx_len, PROMPT):
            runner.step([StepEntry(s, toks[i:i + PROMPT], ())])
    times = []
    launches0 = runner.ops.launches
    for _ in range(max(2, args.steps)):
        torch.cuda.synchronize(); a.record()
        runner.decode_step(slots, rand(B), [0.0] * B, [0] * B)
        b.record(); torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    if runner.ops.profiling:
        runner.ops.take_profile()
        runner.decode_step(slots, rand(B), [0.0] * B, [0] * B)
        print(json.dumps({"case": "decode", "batch": B, "context": ctx_len, "kernel_ms": runner.ops.take_profile()}))
    gbs = (weight_bytes + B * ctx_len * kv_per_token) / min(times) / 1e6
    print(json.dumps({"case": "decode", "shape": args.shape, "batch": B, "context": ctx_len, "layers": cfg.num_hidden_layers,
                      "ms": times, "graphs": bool(args.graphs), "gb_per_s": round(gbs, 1), "frac_of_peak": round(gbs / pk["hbm_gbs"], 3),
                      "launches_per_step": (runner.ops.launches - launches0) // max(2, args.steps)}))
    return 0


def mixed_workload(args, K, W):
    """BASELINE.json's fourth configuration: Llama-3.2-3B layer sizes (28 layers), 32 requests with
    prompt lengths drawn uniformly from 128..2048 (seeded), a token budget of 512 per step (prompt
    portions beside decoded tokens in one forward), 256 new tokens each, through ``Engine``.
    One JSON line: generated tokens/s as ``value`` (wall clock around ``Engine.step()``), tokens/s
    with the prompts, the median time of decode-only and of mixed steps, and the decode-only
    steps against the copy bandwidth."""
    import random
    import statistics

    import torch
    from zllm_b200 import Engine, EngineConfig, LlamaConfig, SamplingParams

    pk, pk_src = peaks()
    cfg = LlamaConfig.from_dict(dict(MODEL, **SHAPES["3b"]))
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg)
    n_req, new_tokens, budget = 32, 256, 512
    rng = random.Random(3)
    lengths = [rng.randint(128, 2048) for _ in range(n_req)]
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    max_len = 2048 + new_tokens + 8
    t0 = time.time()
    eng = Engine(config=cfg, seed=3, random_on_device=True, engine_config=EngineConfig(
        dtype="bfloat16", block_size=BLOCK, num_blocks=n_req * (-(-max_len // BLOCK)) + 8, max_num_seqs=n_req,
        max_num_batched_tokens=budget, max_model_len=max_len, prefix_sharing=False))
    print(f"[bench] model built in {time.time() - t0:.1f} s; weights {weight_bytes / 1e9:.3f} GB", file=sys.stderr, flush=True)
    eng.warm_up(max_batch=n_req, max_context=max_len)

    def run():
        for p in prompts:
            eng.add_request(p, SamplingParams.greedy(max_tokens=new_tokens))
        steps = []                                # (wall ms, decoded rows, prompt tokens, cached positions of the decoded rows)
        torch.cuda.synchronize()
        t_start = last = time.perf_counter()
        n_out = 0
        while eng.has_unfinished():
            cached = sum(len(r.tokens) for r in eng.scheduler.running)
            n_out += len(eng.step())
            now = time.perf_counter()
            ls = eng.last_step
            steps.append(((now - last) * 1e3, ls["decodes"], ls["prompt_tokens"], cached))
            last = now
        torch.cuda.synchronize()
        return time.perf_counter() - t_start, n_out, steps

    clocks = ClockSampler()
    run()                                          # warm-up, twice: a step shape is captured as a graph when it comes a
    run()                                          # second time, so only then has every graph of the workload been made
    clocks.start()
    total_s, n_out, steps = run()
    clk = clocks.stop()
    dec = [s for s in steps if s[2] == 0 and s[1] == n_req]          # all 32 requests decoding, nothing else
    mixed = [s for s in steps if s[2] > 0]
    dec_ms = statistics.median(s[0] for s in dec) if dec else None
    dec_ctx = statistics.median(s[3] for s in dec) if dec else 0
    dec_bytes = weight_bytes + dec_ctx * kv_per_token
    achieved = dec_bytes / (dec_ms / 1e3) / 1e9 if dec_ms else None
    mixed_flops = [2 * (weight_bytes / 2) * (s[1] + s[2]) for s in mixed]     # products only
    line = {
        "metric": "generated tok/s, Llama-3.2-3B shape, bf16, 32 requests, prompts 128-2048 in 512-token portions beside "
                  "decode, 256 new tokens each (random weights)",
        "value": round(n_out / total_s, 1), "unit": "tokens/s", "n_gpus": 1, "steps": len(steps), "warmup": len(steps),
        "ms_per_step": round(total_s * 1e3 / len(steps), 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights N(0,0.02) seed 3)", "impl": "ours",
        "config": {"model": "Llama-3.2-3B-shaped", "layers": cfg.num_hidden_layers, "layers_full": 28,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied": True,
                   "global_batch": n_req, "seq_len": max_len - 8, "prompt_len": "128-2048", "token_budget": budget,
                   "new_tokens": new_tokens, "kv_block": BLOCK, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.2f} GB of weights per step)", "peaks": pk_src},
        "e2e": {"value": round(n_out / total_s, 1), "unit": "tokens/s", "with_prompts": round((n_out + sum(lengths)) / total_s, 1),
                "total_s": round(total_s, 3)},
        "mixed_steps": {"n": len(mixed), "median_ms": round(statistics.median(s[0] for s in mixed), 3) if mixed else None,
                        "median_tflops": round(statistics.median(f / (s[0] / 1e3) / 1e12 for f, s in zip(mixed_flops, mixed)), 1)
                        if mixed else None},
        "decode_steps": {"n": len(dec), "median_ms": round(dec_ms, 3) if dec_ms else None, "rows": n_req},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1) if achieved else None, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4) if achieved else None,
                     "of": "decode-only steps of all 32 requests (median wall time between returns of Engine.step)"},
        "clocks": clk,
    }
    print(json.dumps(line))
    return 0


def cpu_baseline():
    """The plain float32 implementation of the test-suite (tests/plain_llama.py: torch on the CPU,
    the whole sequence recomputed for every token, no cache) timed as the CPU baseline: greedy
    tokens per second on tiny A, tiny B and the two-layer model of Llama-3.2-1B's layer sizes.
    The reference's own CPU path (candle, Q4_K weights, with a cache) cannot be built here."""
    import platform
    import tempfile
    from pathlib import Path

    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama as P
    from configs import TINY, make_model_dir, random_prompt
    from zllm_b200 import LlamaConfig
    from zllm_b200.weights import write_random_model

    cpu = platform.processor() or platform.machine()
    try:
        with open("/proc/cpuinfo") as f:
            cpu = next((l.split(":", 1)[1].strip() for l in f if l.startswith("model name")), cpu)
    except OSError:
        pass
    out = {"impl": "plain CPU implementation (tests/plain_llama.py)", "cpu": cpu, "threads": torch.get_num_threads(),
           "unit": "tokens/s", "results": {}}
    with tempfile.TemporaryDirectory() as tmp:
        cases = [("tiny A", make_model_dir(Path(tmp), "A"), 33, 16), ("tiny B", make_model_dir(Path(tmp), "B"), 33, 16)]
        big = Path(tmp) / "1b2"
        write_random_model(big, LlamaConfig.from_dict(dict(MODEL, num_hidden_layers=2, max_position_embeddings=4096)), 2,
                           "float32", std=0.02)
        cases.append(("Llama-3.2-1B layer sizes, 2 of 16 layers", big, 32, 8))
        for name, d, n_prompt, n_new in cases:
            cfg, w = P.read_model_dir(d)
            prompt = random_prompt(cfg["vocab_size"], n_prompt, 1)
            P.greedy_generate(cfg, w, prompt, 1)
            t = time.perf_counter()
            P.greedy_generate(cfg, w, prompt, n_new)
            dt = time.perf_counter() - t
            out["results"][name] = {"prompt": n_prompt, "new_tokens": n_new, "tokens_per_s": round(n_new / dt, 2)}
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=32)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--config", default="1b", choices=("1b", "8b", "3b-mixed", "cpu-baseline"),
                    help="which of the configurations the numbers are quoted on (default: the 1B headline)")
    ap.add_argument("--case", default=None, choices=("decode", "prefill"),
                    help="run only a small case for a profiler: a few decode steps without graphs, or one prefill")
    ap.add_argument("--context", type=int, default=1024, help="--case decode: cached positions per request")
    ap.add_argument("--tokens", type=int, default=PROMPT, help="--case prefill: tokens of the prompt")
    ap.add_argument("--layers", type=int, default=None, help="--case: fewer layers (profiling only)")
    ap.add_argument("--graphs", action="store_true", help="--case: with CUDA graphs (default off, so that a profiler sees "
                    "every kernel as its own launch)")
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="--case: layer sizes of another Llama shape")
    args = ap.parse_args()

    if args.config == "cpu-baseline":
        return cpu_baseline()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "fankh/zllm is a Rust crate (candle, wgpu, ash): no Rust "
                          "toolchain and no crates offline, so it cannot be installed; its GPU paths need Vulkan or "
                          "wgpu, unavailable on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported (work on several GPUs is "
              "out of its scope)")
        return 2
    K, W = args.steps, max(args.warmup, 3)

    import torch
    from zllm_b200 import Engine, EngineConfig, LlamaConfig, SamplingParams, StepEntry

    if args.case:
        return profile_case(args)
    if args.config == "3b-mixed":
        return mixed_workload(args, K, W)

    pk, pk_src = peaks()
    big = args.config == "8b"
    CONTEXT = 8192 if big else 4096
    shape_name = "Llama-3.1-8B-shaped" if big else "Llama-3.2-1B-shaped"
    seed = 4 if big else 2
    cfg = LlamaConfig.from_dict(dict(MODEL, **SHAPES[args.config]))
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg)
    dev = torch.device("cuda:0")
    max_b = max(64, args.batch)
    n_blocks = max_b * (CONTEXT // BLOCK) + 64
    t0 = time.time()
    eng = Engine(config=cfg, seed=seed, random_on_device=True, engine_config=EngineConfig(
        dtype="bfloat16", block_size=BLOCK, num_blocks=n_blocks, max_num_seqs=max_b, max_num_batched_tokens=PROMPT,
        max_model_len=CONTEXT + 8))
    runner = eng.runner
    print(f"[bench] model built in {time.time() - t0:.1f} s; weights {weight_bytes / 1e9:.3f} GB", file=sys.stderr, flush=True)
    gen = torch.Generator().manual_seed(0)

    def prompt(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    def event_ms(fn):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    def fill(batch, length):
        """``batch`` requests holding ``length`` cached positions each (prompts prefilled in portions)."""
        slots = [runner.admit() for _ in range(batch)]
        for s in slots:
            toks = prompt(length)
            for i in range(0, length, PROMPT):
                runner.step([StepEntry(s, toks[i:i + PROMPT], ())])
        return slots

    def decode_point(batch, steps, warm):
        """tokens/s of ``steps`` decode steps that end at CONTEXT, timed on the device: the steps
        replay one captured graph back to back, each step's sampled token feeding the next."""
        slots = fill(batch, CONTEXT - steps - warm)
        toks = prompt(batch)
        zeros = [0.0] * batch
        seeds = list(range(batch))
        runner.decode_burst(slots, toks, zeros, seeds, warm)          # untimed warm-up (captures the graph)
        ms = event_ms(lambda: runner.decode_burst(slots, toks, zeros, seeds, steps))
        per_replay = max(g["launches"] for g in runner._graphs.values())
        ctx_mean = CONTEXT - steps / 2.0
        for s in slots:
            runner.release(s)
        return batch * steps / (ms / 1e3), ms / steps, per_replay * steps, ctx_mean

    clocks = ClockSampler()
    clocks.start()

    # ---- headline: batch 8 ---------------------------------------------------------------
    B = args.batch
    value, ms_step, launches, ctx_mean = decode_point(B, K, W)
    step_bytes = weight_bytes + B * ctx_mean * kv_per_token
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    # ---- end to end through the Python entry point ------------------------------------------
    # Prompts are prefilled in portions, so the requests start (and would end) decoding a few steps
    # apart: max_tokens leaves room for that, and the warm-up runs until every request decodes.
    slack = 4 * B + 8
    for i in range(B):
        eng.add_request(prompt(CONTEXT - K - W - slack - 2), SamplingParams.greedy(max_tokens=K + W + slack))
    while eng.scheduler.prefilling or eng.scheduler.waiting:
        eng.step()
    def timed_engine_steps():
        """K steps of ``Engine.step()`` by the wall clock; (tokens/s, host-to-device bytes per step).
        The bytes are counted where they are copied (step buffers and block-table rows)."""
        from zllm_b200.engine.batch import StepBuffers
        for _ in range(W):
            eng.step()
        torch.cuda.synchronize()
        up0 = StepBuffers.bytes_uploaded + runner.cache.table_bytes_uploaded
        t1 = time.perf_counter()
        n = 0
        for _ in range(K):
            n += len(eng.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t1
        up = StepBuffers.bytes_uploaded + runner.cache.table_bytes_uploaded - up0
        while eng.has_unfinished():
            eng.step()
        return n / dt, up / K

    e2e_tps, h2d = timed_engine_steps()
    # the same with every step scheduled by the host (no decode step launched ahead): each step
    # then uploads its tokens, positions and slots from pinned memory before it runs
    for i in range(B):
        eng.add_request(prompt(CONTEXT - K - W - slack - 2), SamplingParams.greedy(max_tokens=K + W + slack))
    while eng.scheduler.prefilling or eng.scheduler.waiting:
        eng.step()
    eng.overlap = False
    strict_tps, strict_h2d = timed_engine_steps()
    eng.overlap = True

    # ---- the same with top-k / top-p sampling (the draw among the candidates runs on the device) -------
    for i in range(B):
        eng.add_request(prompt(CONTEXT - K - W - slack - 2),
                        SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=i, max_tokens=K + W + slack))
    while eng.scheduler.prefilling or eng.scheduler.waiting:
        eng.step()
    topp_tps, _ = timed_engine_steps()

    # ---- prefill of 2,048 tokens ------------------------------------------------------------
    s = runner.admit()
    toks = prompt(PROMPT)
    runner.step([StepEntry(s, toks, (PROMPT - 1,))])
    runner.release(s)
    pf = []
    for _ in range(5):
        s = runner.admit()
        pf.append(event_ms(lambda: runner.step([StepEntry(s, toks, (PROMPT - 1,))])))
        runner.release(s)
    pf_ms = sorted(pf)[len(pf) // 2]
    flops = prefill_flops(PROMPT)

    # ---- points -----------------------------------------------------------------------------
    b1, _, _, _ = decode_point(1, min(K, 64), 3)
    b64, ms64, _, ctx64 = decode_point(64, min(K, 64), 3)
    clk = clocks.stop()

    line = {
        "metric": f"decode tok/s, {shape_name.replace('-shaped', '')} shape, bf16, batch {B}, context {CONTEXT} (random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": f"synthetic (uniform random token ids, random weights N(0,0.02) seed {seed})",
        "impl": "ours",
        "config": {"model": shape_name, "layers": cfg.num_hidden_layers, "layers_full": cfg.num_hidden_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": bool(cfg.tie_word_embeddings), "global_batch": B, "seq_len": CONTEXT, "prompt_len": PROMPT,
                   "kv_block": BLOCK, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.2f} GB of weights per step)", "peaks": pk_src},
        # through Engine.step(): while only decoding, the step after the one being read is launched
        # ahead with inputs advanced on the device (an autoregressive step's input IS the last
        # step's output), so a steady-state step copies nothing up; "scheduled" is the same with
        # every step's tokens, positions and slots uploaded from pinned memory before it runs
        "e2e": {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": round(h2d, 1),
                "d2h_bytes_per_step": 4 * B, "scheduled": {"value": round(strict_tps, 1),
                                                           "h2d_bytes_per_step": round(strict_h2d, 1)}},
        "gpu_launches": launches,
        "prefill": {"value": round(PROMPT / (pf_ms / 1e3), 1), "tokens": PROMPT, "ms": round(pf_ms, 3),
                    "frac": round(flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1),
                   f"decode_b{B}_top_p_e2e": round(topp_tps, 1),
                   "decode_b64_hbm_frac": round((weight_bytes + 64 * ctx64 * kv_per_token) / (ms64 / 1e3) / 1e9 / pk["hbm_gbs"], 4)},
        "clocks": clk,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
