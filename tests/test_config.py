"""Configuration and registry (CPU)."""
import json

import pytest

from zllm_b200.config import (EngineConfig, LlamaConfig, architecture, architecture_of, known_architectures,
                              read_config_json)
from zllm_b200.errors import ConfigError
from configs import TINY_A, TINY_B


def test_reads_every_key():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 96, 3, 1, 32)
    assert (c.intermediate_size, c.vocab_size, c.rms_norm_eps, c.rope_theta) == (256, 1000, 1e-6, 500000.0)
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.factor == 8.0
    assert c.rope_scaling.original_max_position_embeddings == 64
    assert c.tie_word_embeddings is False and c.max_position_embeddings == 512


def test_defaults_are_the_documented_ones():
    d = dict(TINY_A)
    for k in ("num_key_value_heads", "head_dim", "rope_theta", "rope_scaling", "tie_word_embeddings"):
        d.pop(k)
    c = LlamaConfig.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads       # absent kv heads means MHA (arch.rs:130)
    assert c.head_dim == 64 // 4                                  # hidden / heads (arch.rs:144-146)
    assert c.rope_theta == 10000.0 and c.rope_scaling is None and c.tie_word_embeddings is False


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "rms_norm_eps", "max_position_embeddings", "architectures"])
def test_missing_mandatory_key_names_the_key(key):
    d = dict(TINY_A)
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(d)


def test_explicit_head_dim_wins_over_division():
    d = dict(TINY_A, head_dim=32)
    assert LlamaConfig.from_dict(d).head_dim == 32


@pytest.mark.parametrize("patch,word", [
    (dict(num_key_value_heads=3), "multiple"), (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"), (dict(rope_scaling={"rope_type": "yarn", "factor": 2}), "yarn"),
    (dict(rope_scaling={"rope_type": "llama3", "factor": 8.0}), "low_freq_factor"),
    (dict(num_hidden_layers=0), "num_hidden_layers"), (dict(rms_norm_eps=0), "rms_norm_eps"),
    (dict(hidden_size=66, head_dim=None), "divisible"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_dict(dict(TINY_A, **patch))


def test_roundtrip_through_config_json(tmp_path):
    c = LlamaConfig.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    raw = read_config_json(tmp_path)
    assert architecture_of(raw).read_config(raw) == c


def test_registry_knows_llama_ignores_case_and_rejects_others():
    assert "LlamaForCausalLM" in known_architectures()
    assert architecture("llamaforcausallm").name == "LlamaForCausalLM"
    with pytest.raises(ConfigError, match="MixtralForCausalLM"):
        architecture("MixtralForCausalLM")
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({})


def test_unreadable_config(tmp_path):
    with pytest.raises(ConfigError, match="cannot read"):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(tmp_path)


def test_model_spec_is_data():
    c = LlamaConfig.from_dict(TINY_B)
    spec = architecture("LlamaForCausalLM").build_spec(c)
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert m.kind == "paged_attention" and m.params["n_kv_heads"] == 1 and m.params["head_dim"] == 32
    assert spec.layers[0].ffn.params == {"hidden_size": 96, "intermediate_size": 256}
    assert spec.layers[0].norm1.params["eps"] == 1e-6
    assert spec.head_name == "lm_head.weight" and spec.head_optional and not spec.tie_head
    assert architecture("LlamaForCausalLM").build_spec(LlamaConfig.from_dict(TINY_A)).tie_head


def test_engine_config_validation():
    EngineConfig().validate()
    with pytest.raises(ConfigError, match="dtype"):
        EngineConfig(dtype="float16").validate()
    with pytest.raises(ConfigError, match="block_size"):
        EngineConfig(block_size=0).validate()
