"""The oracle is stated twice, by different routes, and the two must agree (CPU).

``plain_llama.py``: torch, whole sequences, half-split rotation of the folder's weights, the
llama3 blend on theta_j.  ``plain_reference_path.py``: NumPy, token by token against a growing
cache, the reference's interleaved rotation on converter-permuted weights, a table of frequency
divisors, two-pass or online softmax.  In double precision they agree to 1e-9, which leaves no
room for a different reading of the rotary pairing, the llama3 rule, the group-to-head map, the
mask, eps, SiLU or the tied head; in float32 ``plain_llama.py`` stays within 2e-5 of that."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama as P
import plain_reference_path as R
from configs import TINY, make_model_dir, random_prompt


@pytest.mark.parametrize("name", sorted(TINY))
def test_the_two_plain_statements_agree(tmp_path, name):
    d = make_model_dir(tmp_path, name)
    cfg, w = P.read_model_dir(d)
    cfg2, w2 = R.read_folder(d)
    toks = random_prompt(cfg["vocab_size"], 37, 11)
    ref = R.logits_token_by_token(cfg2, w2, toks)
    scale = float(np.abs(ref).max())
    a64 = P.forward_all_positions(cfg, w, toks, dtype=torch.float64).numpy()
    assert float(np.abs(a64 - ref).max()) < 1e-9 * max(1.0, scale)
    a32 = P.forward_all_positions(cfg, w, toks).double().numpy()
    assert float(np.abs(a32 - ref).max()) < 2e-5
    assert (a32.argmax(-1) == ref.argmax(-1)).all()
    # the online softmax of the reference's shaders is the same function
    on = R.logits_token_by_token(cfg2, w2, toks[:19], online=True)
    assert float(np.abs(on - ref[:19]).max()) < 1e-9 * max(1.0, scale)


def test_the_two_statements_agree_on_a_window(tmp_path):
    d = make_model_dir(tmp_path, "A")
    cfg, w = P.read_model_dir(d)
    cfg2, w2 = R.read_folder(d)
    toks = random_prompt(cfg["vocab_size"], 30, 12)
    a = P.forward_all_positions(cfg, w, toks, dtype=torch.float64, window=7).numpy()
    b = R.logits_token_by_token(cfg2, w2, toks, window=7)
    assert float(np.abs(a - b).max()) < 1e-9
    assert float(np.abs(a - P.forward_all_positions(cfg, w, toks, dtype=torch.float64).numpy()).max()) > 1e-4


def test_a_folder_without_a_head_tensor_is_tied_in_both(tmp_path):
    from zllm_b200.weights import write_safetensors
    d = make_model_dir(tmp_path, "B")
    w = P.read_safetensors(d / "model.safetensors")
    del w["lm_head.weight"]
    write_safetensors(d / "model.safetensors", w)
    cfg, w1 = P.read_model_dir(d)                   # the flag still says "untied"
    cfg2, w2 = R.read_folder(d)
    toks = random_prompt(cfg["vocab_size"], 9, 13)
    a = P.forward_all_positions(cfg, w1, toks, dtype=torch.float64).numpy()
    assert float(np.abs(a - R.logits_token_by_token(cfg2, w2, toks)).max()) < 1e-9


@pytest.mark.parametrize("name", sorted(TINY))
def test_golden_numbers(tmp_path, name):
    """tests/golden/tiny_logits.json (made by tests/golden/make_golden.py) pins the statements,
    the random-weights mode and the reading of the configurations against drift."""
    g = json.loads((Path(__file__).parent / "golden" / "tiny_logits.json").read_text())[name]
    cfg, w = P.read_model_dir(make_model_dir(tmp_path, name))
    lg = P.forward_all_positions(cfg, w, g["tokens"])[-1]
    assert float((lg[:len(g["first"])].double() - torch.tensor(g["first"], dtype=torch.float64)).abs().max()) < 2e-5
    assert int(lg.argmax()) == g["argmax"] and abs(float(lg.max()) - g["max"]) < 2e-5
