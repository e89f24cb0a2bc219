"""The dense Llama decoder as a :class:`ModelSpec`.

Every layer: pre-norm block of grouped-query attention with rotary embedding (half-split
pairing, the layout of Hugging Face checkpoints; optional llama3 frequency scaling) and a
SwiGLU feed-forward, RMSNorm throughout, embeddings optionally tied to the head
(crates/allpaca-core/src/model.rs:8195-8802 is the reference's forward of this
architecture; tensor names: crates/allpaca-safetensors/src/names.rs:26-102).
"""
from __future__ import annotations

from ..config.model_config import ConfigError, LlamaConfig
from ..parts import LayerRun, ModelSpec, PartSpec
from .registry import register_architecture


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    if cfg.head_dim % 16 != 0 or cfg.head_dim > 256:
        # what the attention kernels are built for: said when the model is described, before
        # any weight is read or any kernel is compiled
        raise ConfigError(f"head_dim {cfg.head_dim} is not one the attention kernels take "
                          f"(multiples of 16 up to 256)")
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    rope = PartSpec("rope", {
        "head_dim": cfg.head_dim, "theta": cfg.rope_theta, "pairing": "half",
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None})
    mixer = PartSpec("gqa_attention", {
        "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
        "position": rope, "window": None})
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                              "intermediate_size": cfg.intermediate_size})
    block = PartSpec("prenorm", {
        "hidden_size": cfg.hidden_size, "mixer": mixer, "feed_forward": ffn,
        "mixer_norm": norm, "feed_forward_norm": norm,
        "mixer_prefix": "self_attn.", "feed_forward_prefix": "mlp.",
        "mixer_norm_prefix": "input_layernorm.",
        "feed_forward_norm_prefix": "post_attention_layernorm."})
    n = cfg.num_hidden_layers
    return ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        layers=tuple(block for _ in range(n)),
        layer_prefixes=tuple(f"model.layers.{i}." for i in range(n)),
        order=tuple(LayerRun(i) for i in range(n)),
        final_norm=norm,
        tie_word_embeddings=cfg.tie_word_embeddings,
        max_position_embeddings=cfg.max_position_embeddings)


register_architecture(("LlamaForCausalLM", "llama"), LlamaConfig, llama_spec)
