"""LlamaForCausalLM: the dense Llama decoder as a list of parts.

Every layer: RMSNorm -> grouped-query attention with rotary encoding ->
residual -> RMSNorm -> SiLU-gated feed-forward -> residual; then a final
RMSNorm and the output head, tied to the embedding or not (zllm
src/backend/candle/quantized_llama_fork.rs:920-987; layer contents 433-537,
394-400).  Tensor names are those of a safetensors model folder; the
reference's GGUF names for the same tensors are listed at fork.rs:755-791.
Rotary pairing is half-split, which is what unpermuted safetensors weights use
(the reference rotates interleaved pairs because GGUF converters permute the
rows of Wq and Wk, src/backend/arch.rs:25-35).
"""
from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunEntry


def _as_ids(eos) -> tuple:
    """config.json gives one end-of-text id or a list of them (or none)."""
    if isinstance(eos, bool) or eos is None:
        return ()
    if isinstance(eos, int):
        return (eos,)
    return tuple(int(e) for e in eos)


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    rotary = PartSpec("rotary", {
        "rot_dim": cfg.head_dim,
        "theta": cfg.rope_theta,
        "max_position": cfg.max_position_embeddings,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
        "interleaved": False,
    })
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            mixer=PartSpec("paged_attention", {
                "hidden_size": cfg.hidden_size,
                "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "position_encoding": rotary,
            }),
            ffn=PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size}),
            norm1=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}),
            norm2=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}),
            arrangement="pre_norm",
            tensor_names={
                "norm1.weight": p + "input_layernorm.weight",
                "mixer.q_proj": p + "self_attn.q_proj.weight",
                "mixer.k_proj": p + "self_attn.k_proj.weight",
                "mixer.v_proj": p + "self_attn.v_proj.weight",
                "mixer.o_proj": p + "self_attn.o_proj.weight",
                "norm2.weight": p + "post_attention_layernorm.weight",
                "ffn.gate_proj": p + "mlp.gate_proj.weight",
                "ffn.up_proj": p + "mlp.up_proj.weight",
                "ffn.down_proj": p + "mlp.down_proj.weight",
            },
        ))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_position=cfg.max_position_embeddings,
        layers=layers,
        run_order=[RunEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}),
        embedding_name="model.embed_tokens.weight",
        final_norm_names={"weight": "model.norm.weight"},
        # the head is tied iff the folder has no lm_head.weight (fork.rs:761-764); the flag only
        # decides what the random-weights mode writes
        head_name="lm_head.weight",
        head_optional=True,
        tie_head=bool(cfg.tie_word_embeddings),
        # older checkpoints store each layer's rotary frequencies; they follow from the configuration
        ignored_tensors=("*.rotary_emb.inv_freq",),
        stop_token_ids=_as_ids(cfg.eos_token_id),
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, build_llama_spec)
