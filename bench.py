#!/usr/bin/env python3
"""Benchmark: decoded tokens per second of the Llama-3.2-1B-shaped model (random weights,
bfloat16) on one B200, with prefill throughput, roofline fractions and end-to-end numbers.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

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
        cuda_graphs=False))
    gen = torch.Generator().manual_seed(0)
    rand = lambda n: torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.case == "prefill":
        toks = rand(args.tokens)
        times = []
        for _ in range(max(2, args.steps)):
            s = runner.admit()
            torch.cuda.synchronize(); a.record()
            runner.step([StepEntry(s, toks, (len(toks) - 1,))])
            b.record(); torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
            runner.release(s)
        best = min(times)
        print(json.dumps({"case": "prefill", "shape": args.shape, "tokens": args.tokens, "layers": cfg.num_hidden_layers,
                          "ms": times, "tflops": round(prefill_flops(args.tokens) / best / 1e9, 1),
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
    gbs = (weight_bytes + B * ctx_len * kv_per_token) / min(times) / 1e6
    print(json.dumps({"case": "decode", "shape": args.shape, "batch": B, "context": ctx_len, "layers": cfg.num_hidden_layers,
                      "ms": times, "graphs": False, "gb_per_s": round(gbs, 1), "frac_of_peak": round(gbs / pk["hbm_gbs"], 3),
                      "launches_per_step": (runner.ops.launches - launches0) // max(2, args.steps)}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--case", default=None, choices=("decode", "prefill"),
                    help="run only a small case for a profiler: a few decode steps without graphs, or one prefill")
    ap.add_argument("--context", type=int, default=1024, help="--case decode: cached positions per request")
    ap.add_argument("--tokens", type=int, default=PROMPT, help="--case prefill: tokens of the prompt")
    ap.add_argument("--layers", type=int, default=None, help="--case: fewer layers (profiling only)")
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="--case: layer sizes of another Llama shape")
    args = ap.parse_args()

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

    pk, pk_src = peaks()
    cfg = LlamaConfig.from_dict(MODEL)
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg)
    dev = torch.device("cuda:0")
    max_b = max(64, args.batch)
    n_blocks = max_b * (CONTEXT // BLOCK) + 64
    t0 = time.time()
    eng = Engine(config=cfg, seed=2, random_on_device=True, engine_config=EngineConfig(
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
    for _ in range(W):
        eng.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    n_tok = 0
    for _ in range(K):
        n_tok += len(eng.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t1
    g8 = next(g for k, g in runner._graphs.items() if k[0] == 8) if B == 8 else None
    h2d = (g8["buf"].total * 4) if g8 else None
    while eng.has_unfinished():
        eng.step()

    # ---- the same with top-k / top-p sampling (the draw among the candidates runs on the device) -------
    for i in range(B):
        eng.add_request(prompt(CONTEXT - K - W - slack - 2),
                        SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=i, max_tokens=K + W + slack))
    while eng.scheduler.prefilling or eng.scheduler.waiting:
        eng.step()
    for _ in range(W):
        eng.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    n_tok_p = 0
    for _ in range(K):
        n_tok_p += len(eng.step())
    torch.cuda.synchronize()
    topp_s = time.perf_counter() - t1
    while eng.has_unfinished():
        eng.step()

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
        "metric": "decode tok/s, Llama-3.2-1B shape, bf16, batch 8, context 4096 (random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights N(0,0.02) seed 2)",
        "impl": "ours",
        "config": {"model": "Llama-3.2-1B-shaped", "layers": cfg.num_hidden_layers, "layers_full": 16,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": True, "global_batch": B, "seq_len": CONTEXT, "prompt_len": PROMPT, "kv_block": BLOCK,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (2.47 GB of weights per step)",
                   "peaks": pk_src},
        "e2e": {"value": round(n_tok / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * B},
        "gpu_launches": launches,
        "prefill": {"value": round(PROMPT / (pf_ms / 1e3), 1), "tokens": PROMPT, "ms": round(pf_ms, 3),
                    "frac": round(flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1),
                   "decode_b8_top_p_e2e": round(n_tok_p / topp_s, 1),
                   "decode_b64_hbm_frac": round((weight_bytes + 64 * ctx64 * kv_per_token) / (ms64 / 1e3) / 1e9 / pk["hbm_gbs"], 4)},
        "clocks": clk,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
