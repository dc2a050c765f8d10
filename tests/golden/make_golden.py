"""Writes ``tiny_logits.json``: for each tiny configuration a short prompt's logits at its
last position (the first 24 vocabulary entries, the largest entry and its index), computed in
double precision by ``tests/plain_reference_path.py``.

The reference (fankh/zllm) is Rust and can be neither imported nor compiled where this suite
runs, and it ships no golden numbers, so these are NOT the reference's outputs: they are the
outputs of the plain statements at the time both agreed, kept so that a later change to
either statement, to the random-weights mode or to the reading of a configuration shows.

    python tests/golden/make_golden.py          # rewrites tests/golden/tiny_logits.json
"""
import json
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path[:0] = [str(HERE.parent), str(HERE.parent.parent)]

import plain_reference_path as R          # noqa: E402
from configs import TINY, make_model_dir, random_prompt          # noqa: E402

N_TOKENS = 20
N_KEPT = 24


def compute():
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name in sorted(TINY):
            cfg, w = R.read_folder(make_model_dir(Path(tmp), name))
            toks = random_prompt(cfg["vocab_size"], N_TOKENS, 100 + ord(name))
            lg = R.logits_token_by_token(cfg, w, toks)[-1]
            out[name] = {"tokens": toks, "first": [float(v) for v in lg[:N_KEPT]],
                         "argmax": int(lg.argmax()), "max": float(lg.max())}
    return out


if __name__ == "__main__":
    (HERE / "tiny_logits.json").write_text(json.dumps(compute(), indent=1))
    print("wrote", HERE / "tiny_logits.json")
