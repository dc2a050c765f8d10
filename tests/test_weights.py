"""Weights: container, checks, random mode (CPU)."""
import json

import pytest
import torch

from zllm_b200.config import LlamaConfig, architecture
from zllm_b200.errors import ModelError
from zllm_b200.models import expected_tensors
from zllm_b200.weights import (SafetensorsFile, load_checked, open_model_files, target_dtype, write_random_model,
                               write_safetensors)
from configs import TINY_A, TINY_B, make_model_dir
import plain_llama as P


def _expected(cfg_dict):
    c = LlamaConfig.from_dict(cfg_dict)
    return expected_tensors(architecture(c.architecture).build_spec(c))


def test_container_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3)}
    write_safetensors(tmp_path / "x.safetensors", t)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(f.keys()) == ["a", "b", "c"]
    for k, v in t.items():
        assert f.meta(k) == (v.dtype, tuple(v.shape))
        assert torch.equal(f.tensor(k), v)
    # the plain implementation's own reader agrees (it shares no code with the package)
    own = P.read_safetensors(tmp_path / "x.safetensors")
    assert torch.equal(own["a"], t["a"]) and torch.equal(own["b"], t["b"].float())


def test_expected_names_and_shapes():
    e = _expected(TINY_B)
    assert e["model.embed_tokens.weight"].shape == (1000, 96)
    assert e["lm_head.weight"].shape == (1000, 96)
    assert e["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert e["model.layers.0.mlp.down_proj.weight"].shape == (96, 256)
    assert "lm_head.weight" not in _expected(TINY_A)           # tied by its flag: random mode writes none
    assert len(e) == 2 + 1 + 3 * 9


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_dir(tmp_path, "A")
    w = P.read_safetensors(d / "model.safetensors")
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    w["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(8)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)      # a harmless extra: not reported
    write_safetensors(d / "model.safetensors", w)
    with pytest.raises(ModelError) as ei:
        load_checked(d, _expected(TINY_A), torch.float32, "cpu", ignored=("*.rotary_emb.inv_freq",))
    msg = str(ei.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "q_norm.weight" in msg and "unexpected tensors (1)" in msg and "rotary_emb.inv_freq" not in msg
    assert "expected [64, 64], found [64, 63]" in msg and "missing tensors (2)" in msg


def test_missing_folder_and_bad_file(tmp_path):
    with pytest.raises(ModelError, match="neither"):
        open_model_files(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"\x05\x00")
    with pytest.raises(ModelError, match="invalid safetensors"):
        open_model_files(tmp_path)


def test_dtype_policy():
    bf, f32 = torch.bfloat16, torch.float32
    assert target_dtype(bf, "matrix", bf) == bf
    assert target_dtype(f32, "vector", bf) == f32          # a tensor stored in 32-bit stays so
    assert target_dtype(bf, "vector", bf) == bf
    assert target_dtype(f32, "matrix", bf) == bf           # tensor-core operands are bfloat16
    assert target_dtype(bf, "matrix", f32) == f32          # the 32-bit path widens everything
    assert target_dtype(torch.int64, "int", bf) == torch.int32


def test_random_mode_is_seeded_and_independent_of_order(tmp_path):
    c = LlamaConfig.from_dict(TINY_A)
    a = write_random_model(tmp_path / "a", c, 7, "float32", std=0.02, norm_std=0.1)
    b = write_random_model(tmp_path / "b", c, 7, "float32", std=0.02, norm_std=0.1)
    c2 = write_random_model(tmp_path / "c", c, 8, "float32", std=0.02, norm_std=0.1)
    wa, wb, wc = (P.read_safetensors(x / "model.safetensors") for x in (a, b, c2))
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    assert not torch.equal(wa["model.embed_tokens.weight"], wc["model.embed_tokens.weight"])
    assert abs(float(wa["model.embed_tokens.weight"].std()) - 0.02) < 2e-3
    assert abs(float(wa["model.norm.weight"].mean()) - 1.0) < 0.1
    cfg = json.loads((a / "config.json").read_text())
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["num_key_value_heads"] == 2
    # the same tensor in a model with more layers has the same values (seeded by name)
    c3 = LlamaConfig.from_dict(dict(TINY_A, num_hidden_layers=3))
    wd = P.read_safetensors(write_random_model(tmp_path / "d", c3, 7, "float32", std=0.02, norm_std=0.1) / "model.safetensors")
    assert torch.equal(wd["model.layers.1.mlp.up_proj.weight"], wa["model.layers.1.mlp.up_proj.weight"])


def test_bfloat16_folder_loads_as_stored(tmp_path):
    d = make_model_dir(tmp_path, "B", "bfloat16")
    t = load_checked(d, _expected(TINY_B), torch.bfloat16, "cpu")
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    t32 = load_checked(d, _expected(TINY_B), torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["lm_head.weight"], t["lm_head.weight"].float())


# ---- the output head is tied iff the folder has no head tensor (fork.rs:761-764) -----------

def _load_model(d, cfg_dict):
    """The tensors as the engine loads them, and the model with them (CPU, no kernels run)."""
    from zllm_b200.models import DecoderModel, Runtime
    c = LlamaConfig.from_dict(cfg_dict)
    spec = architecture(c.architecture).build_spec(c)
    m = DecoderModel(spec, Runtime(torch.float32, torch.device("cpu"), None))
    t = load_checked(d, m.required_tensors(), torch.float32, "cpu", optional=m.optional_tensors(),
                     ignored=spec.ignored_tensors)
    m.load_weights(t)
    return m


def test_head_is_tied_when_the_tensor_is_absent_whatever_the_flag_says(tmp_path):
    import warnings
    d = make_model_dir(tmp_path, "B")                           # untied: lm_head.weight is there
    w = P.read_safetensors(d / "model.safetensors")
    with warnings.catch_warnings():
        warnings.simplefilter("error")                          # flag and folder agree: no warning
        m = _load_model(d, TINY_B)
    assert m.head is not m.embedding and torch.equal(m.head, w["lm_head.weight"])
    del w["lm_head.weight"]
    write_safetensors(d / "model.safetensors", w)
    with pytest.warns(UserWarning, match="untied.*lack"):
        m = _load_model(d, TINY_B)                              # flag false, tensor absent: tied, with a warning
    assert m.head is m.embedding
    # and the plain implementation reads the same folder the same way
    cfg, pw = P.read_model_dir(d)
    assert "lm_head.weight" not in pw


def test_head_tensor_that_is_present_is_used_although_the_flag_says_tied(tmp_path):
    d = make_model_dir(tmp_path, "A")                           # tied by its flag: no lm_head.weight
    w = P.read_safetensors(d / "model.safetensors")
    m = _load_model(d, TINY_A)
    assert m.head is m.embedding
    w["lm_head.weight"] = torch.randn(512, 64)
    write_safetensors(d / "model.safetensors", w)
    with pytest.warns(UserWarning, match="tied.*hold"):
        m = _load_model(d, TINY_A)
    assert torch.equal(m.head, w["lm_head.weight"]) and m.head is not m.embedding
    w["lm_head.weight"] = torch.randn(512, 63)                  # present but mis-shaped: reported like any other
    write_safetensors(d / "model.safetensors", w)
    with pytest.raises(ModelError, match=r"lm_head.weight: expected \[512, 64\], found \[512, 63\]"):
        _load_model(d, TINY_A)


# ---- sharded folders ------------------------------------------------------------------------

def _shard(d, n_first):
    """Rewrite the folder's single file as two shards and an index; returns the tensors."""
    w = P.read_safetensors(d / "model.safetensors")
    names = list(w)
    parts = {"model-00001-of-00002.safetensors": names[:n_first], "model-00002-of-00002.safetensors": names[n_first:]}
    for fname, ns in parts.items():
        write_safetensors(d / fname, {n: w[n] for n in ns})
    (d / "model.safetensors.index.json").write_text(json.dumps(
        {"metadata": {"total_size": 0}, "weight_map": {n: f for f, ns in parts.items() for n in ns}}))
    (d / "model.safetensors").unlink()
    return w, parts


def test_sharded_folder_loads_like_the_single_file(tmp_path):
    d = make_model_dir(tmp_path, "B")
    w, parts = _shard(d, 11)
    m = _load_model(d, TINY_B)
    assert torch.equal(m.head, w["lm_head.weight"]) and torch.equal(m.embedding, w["model.embed_tokens.weight"])
    t = load_checked(d, _expected(TINY_B), torch.float32, "cpu")
    assert set(t) == set(w) and all(torch.equal(t[n], w[n]) for n in w)
    where = open_model_files(d)
    assert {f.path.name for f in where.values()} == set(parts)


def test_index_that_names_a_tensor_its_shard_lacks(tmp_path):
    d = make_model_dir(tmp_path, "B")
    w, parts = _shard(d, 11)
    first = "model-00001-of-00002.safetensors"
    gone = parts[first][3]
    write_safetensors(d / first, {n: w[n] for n in parts[first] if n != gone})
    with pytest.raises(ModelError, match="places .* which does not hold it") as ei:
        open_model_files(d)
    assert gone in str(ei.value)
    # a shard the index names and the folder lacks
    (d / "model-00002-of-00002.safetensors").unlink()
    write_safetensors(d / first, {n: w[n] for n in parts[first]})
    with pytest.raises(ModelError, match="cannot open model file"):
        open_model_files(d)
