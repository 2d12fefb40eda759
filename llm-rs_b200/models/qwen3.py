"""Qwen3 dense decoder as a ``ModelSpec``.

Layer by layer as the reference's graph builder emits it
(llm-core/src/graph/builder.rs:74-297,408-437): RMSNorm -> grouped-query attention with
per-head q/k RMSNorm and rotary position encoding -> residual -> RMSNorm -> SwiGLU ->
residual; final RMSNorm; output head tied to the embedding or not. Two points differ
from the reference on purpose: the rotation pairs (x[i], x[i+d/2]) as the published
weights assume, and the q/k norms are always applied (the reference only finds them
under their GGUF-derived names, llm-core/src/graph/scan.rs:159-176).
"""
from __future__ import annotations

from ..config import ArchitectureEntry, Qwen3Config, register_architecture
from ..parts import LayerSpec, ModelSpec, PartSpec, RunStep


# The tensor names of the architecture's checkpoints (the reference's scan knows the same ones,
# llm-core/src/graph/scan.rs:105-110,152-171); the parts themselves know only roles.
EMBEDDING, FINAL_NORM, HEAD = "model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"
ATTENTION_SCOPE, ATTENTION_NAMES = "self_attn.", {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj",
                                                  "q_norm": "q_norm", "k_norm": "k_norm"}
FEED_FORWARD_SCOPE, FEED_FORWARD_NAMES = "mlp.", {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    H = cfg.hidden_size
    norm = lambda name: PartSpec("rmsnorm", {"dim": H, "eps": cfg.rms_norm_eps, "name": name})
    layers = []
    for i in range(cfg.num_hidden_layers):
        if cfg.no_rope_layers[i]:
            position = PartSpec("none", {"head_dim": cfg.head_dim})
        else:
            position = PartSpec("rope_half", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
        mixer = PartSpec("gqa_attention", {
            "hidden_size": H, "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "position": position, "qk_norm": True,
            "qk_norm_eps": cfg.rms_norm_eps, "bias": cfg.attention_bias, "window": cfg.layer_windows[i],
            "names": ATTENTION_NAMES})
        ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": cfg.intermediate_size,
                                  "names": FEED_FORWARD_NAMES})
        prefix = f"model.layers.{i}."
        layers.append(LayerSpec(
            prefix=prefix, block=PartSpec("prenorm"),
            mixer=PartSpec(mixer.kind, {**mixer.params}), feed_forward=ffn,
            mixer_norm=norm("input_layernorm.weight"), feed_forward_norm=norm("post_attention_layernorm.weight"),
            mixer_scope=ATTENTION_SCOPE, feed_forward_scope=FEED_FORWARD_SCOPE))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab_size, layers=tuple(layers),
        run_order=tuple(RunStep(i) for i in range(cfg.num_hidden_layers)),
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": EMBEDDING}),
        final_norm=PartSpec("rmsnorm", {"dim": H, "eps": cfg.rms_norm_eps, "name": FINAL_NORM}),
        lm_head=PartSpec("linear_head", {
            "vocab_size": cfg.vocab_size, "hidden_size": H, "name": HEAD,
            "tied_to": EMBEDDING if cfg.tie_word_embeddings else ""}),
        max_positions=cfg.max_position_embeddings, eos_token_ids=tuple(cfg.eos_token_ids))


register_architecture(ArchitectureEntry(
    name=Qwen3Config.architecture, model_type=Qwen3Config.model_type,
    config_cls=Qwen3Config, build_spec=build_spec), replace=True)
