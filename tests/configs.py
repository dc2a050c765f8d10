"""The tiny configurations of the suite and helpers to make model folders and prompts.

Tiny A and tiny B differ in every size and option (head counts and groups, sizes
that are no power of two, layers, vocabulary, eps, rope base and scaling, tied or
untied head, page size).  Tiny C has head size 64 and a 4:1 group so that the
tensor-core attention and product kernels run inside the whole-engine tests too; tiny D has
head size 128 (heads x head size larger than the width), a page of 32 positions and an odd
vocabulary.  Tiny E has head size 80 (the mma.sync attention kernels, key rows that share
cache lines), a 3:1 group and linear rope scaling.
"""
from __future__ import annotations

import torch

from zllm_b200.config import LlamaConfig

TINY_A = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=192, vocab_size=512, rms_norm_eps=1e-5,
              rope_theta=10000.0, rope_scaling=None, max_position_embeddings=256, tie_word_embeddings=True)
TINY_B = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
              num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=1000, rms_norm_eps=1e-6,
              rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64),
              max_position_embeddings=512, tie_word_embeddings=False)
TINY_C = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=320, num_attention_heads=8,
              num_key_value_heads=2, head_dim=64, intermediate_size=448, vocab_size=1536, rms_norm_eps=1e-5,
              rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=128),
              max_position_embeddings=1024, tie_word_embeddings=True)

TINY_D = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
              num_key_value_heads=2, head_dim=128, intermediate_size=384, vocab_size=777, rms_norm_eps=1e-5,
              rope_theta=10000.0, rope_scaling=None, max_position_embeddings=1024, tie_word_embeddings=False)

# head size 80: a key row of 160 bytes is no whole number of 128-byte cache lines and none of the
# TMA or tcgen05 attention kernels takes it; a 3:1 group, linear rope scaling, an odd width
TINY_E = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=168, num_attention_heads=6,
              num_key_value_heads=2, head_dim=80, intermediate_size=200, vocab_size=641, rms_norm_eps=3e-6,
              rope_theta=100000.0, rope_scaling=dict(rope_type="linear", factor=2.0),
              max_position_embeddings=768, tie_word_embeddings=False)

# name -> (config dict, page size, weight seed, std of matrices)
TINY = {
    "A": (TINY_A, 16, 0, 0.02),
    "B": (TINY_B, 8, 1, 0.05),
    "C": (TINY_C, 16, 2, 0.04),
    "D": (TINY_D, 32, 3, 0.05),
    "E": (TINY_E, 16, 4, 0.05),
}


# Weight scales for the generation tests: large enough that greedy choices are no rounding ties
# in float32, small enough that the bfloat16 engine stays within ~2 % of the largest logit (the
# error grows with the scale: tiny B at 0.3 is 9 % off in places, at 0.1 under 2 %).
GEN_STD = {"A": 0.15, "B": 0.1, "C": 0.1, "D": 0.1, "E": 0.1}


def typed(name: str) -> LlamaConfig:
    return LlamaConfig.from_dict(TINY[name][0])


def make_model_dir(tmp_path, name: str, dtype: str = "float32", std=None):
    """Write the tiny model ``name`` under ``tmp_path``; returns the folder."""
    from zllm_b200.weights import write_random_model

    cfg, _, seed, s = TINY[name]
    d = tmp_path / f"tiny{name}_{dtype}"
    if not (d / "model.safetensors").exists():
        write_random_model(d, LlamaConfig.from_dict(cfg), seed, dtype, std=std if std is not None else s, norm_std=0.1)
    return d


def random_prompt(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
