"""Command line in the manner of ``zllm generate`` (zllm src/main.rs:25-41,500-659).

    python -m zllm_b200 generate --model DIR --prompt STR|--prompt-ids 1,2,3 \
        [--tokenizer PATH] [--max-tokens 128] [--temperature 0.7] [--top-k 50] [--top-p 0.9] [--seed 0]

Option names, meanings and defaults are the reference's (main.rs:27-40:
--model/-m, --tokenizer/-t "", --prompt/-p, --max-tokens 128, --temperature 0.7,
--top-k 50, --top-p 0.9); it prints the prompt, the generated text as it comes,
and ``--- N tokens in T s (X tok/s) ---`` (main.rs:641).  A model folder takes the
place of the GGUF file; ``tokenizer.json`` beside the model is used when
--tokenizer is empty (main.rs:514-528).  Without any tokenizer, give --prompt-ids
and token ids are printed.  ``random`` writes a model folder with random weights.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def _load_tokenizer(model_dir: Path, explicit: str):
    path = Path(explicit) if explicit else model_dir / "tokenizer.json"
    if not path.exists():
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(str(path))


def cmd_generate(args) -> int:
    from . import Engine, SamplingParams, ZllmError

    model_dir = Path(args.model)
    tok = _load_tokenizer(model_dir, args.tokenizer)
    if args.prompt_ids:
        prompt_ids = [int(t) for t in args.prompt_ids.replace(" ", "").split(",") if t]
    elif args.prompt is not None:
        if tok is None:
            print("zllm generate: --prompt needs a tokenizer (tokenizer.json beside the model or --tokenizer); "
                  "use --prompt-ids otherwise", file=sys.stderr)
            return 2
        prompt_ids = tok.encode(args.prompt).ids
    else:
        print("zllm generate: give --prompt or --prompt-ids", file=sys.stderr)
        return 2
    try:
        eng = Engine(str(model_dir), dtype=args.dtype, max_num_seqs=1, block_size=args.block_size,
                     max_model_len=args.max_seq_len)
        stops = list(eng.runner.spec.stop_token_ids)        # the architecture's end-of-text ids
        params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed,
                                max_tokens=args.max_tokens, stop_token_ids=tuple(stops))
        rid = eng.add_request(prompt_ids, params)
    except ZllmError as e:
        print(f"zllm generate: {e}", file=sys.stderr)
        return 1
    if args.prompt is not None and not args.prompt_ids:
        print(args.prompt, end="", flush=True)
    else:
        print("prompt ids:", ",".join(map(str, prompt_ids)))
    generated = []
    printed = 0
    start = time.time()
    while eng.has_unfinished():
        for _, t, done in eng.step():
            if done and t in stops:
                break                       # the reference stops before printing a stop token (main.rs:616-618)
            generated.append(t)
            if tok is not None:
                text = tok.decode(generated)   # decode the whole tail, print the new suffix (main.rs:624-634)
                print(text[printed:], end="", flush=True)
                printed = len(text)
            else:
                print(t, end=" ", flush=True)
    elapsed = time.time() - start
    print()
    print()
    print(f"--- {len(generated)} tokens in {elapsed:.2f}s ({len(generated) / max(elapsed, 1e-9):.1f} tok/s) ---")
    return 0


def cmd_random(args) -> int:
    from .config import architecture_of
    from .weights import write_random_model

    raw = json.loads(Path(args.config).read_text())
    cfg = architecture_of(raw).read_config(raw)
    out = write_random_model(args.out, cfg, args.seed, args.dtype, std=args.std, norm_std=args.norm_std)
    print(f"wrote {out}/config.json and {out}/model.safetensors (seed {args.seed}, {args.dtype})")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="zllm", description="zllm_b200 -- Llama inference engine for one B200")
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="Generate text from a prompt")
    g.add_argument("-m", "--model", required=True, help="model folder (config.json + model.safetensors)")
    g.add_argument("-t", "--tokenizer", default="", help="tokenizer.json (default: beside the model)")
    g.add_argument("-p", "--prompt", default=None)
    g.add_argument("--prompt-ids", default="", help="comma-separated token ids instead of --prompt")
    g.add_argument("--max-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.7)
    g.add_argument("--top-k", type=int, default=50)
    g.add_argument("--top-p", type=float, default=0.9)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    g.add_argument("--block-size", type=int, default=16)
    g.add_argument("--max-seq-len", type=int, default=None, help="cap of the context (reference: model.max_seq_len)")
    g.set_defaults(fn=cmd_generate)
    r = sub.add_parser("random", help="Write a model folder with random weights from a config.json and a seed")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    r.add_argument("--std", type=float, default=None)
    r.add_argument("--norm-std", type=float, default=0.0)
    r.set_defaults(fn=cmd_random)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
