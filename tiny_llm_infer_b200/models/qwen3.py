"""Qwen3 dense as data: which registered parts each layer is made of.

Per layer (reference: model/src/qwen3_layers.cpp:207-243 for the tensor names,
model/src/qwen3_paged_batch.cpp:144-302 for the arrangement): RMSNorm, grouped-query
attention with per-head q/k norm (same eps as the other norms) and rotate-half rotary
encoding, RMSNorm, SwiGLU feed-forward; pre-norm residual block.  Layers listed as
sliding in the configuration get the window; the others keep every key.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.qwen3 import Qwen3Config
from ..parts.spec import ExecEntry, LayerSpec, ModelDescription, PartSpec


def describe_qwen3(cfg: Qwen3Config) -> ModelDescription:
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps)
        layers.append(LayerSpec("prenorm", {
            "norm1": PartSpec("rmsnorm", norm, p + "input_layernorm."),
            "mixer": PartSpec("gq_attention", dict(
                hidden_size=cfg.hidden_size, q_heads=cfg.num_attention_heads,
                kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                qk_norm_eps=cfg.rms_norm_eps,
                position=PartSpec("rotary_half", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta)),
                window=cfg.window_of_layer(i)), p + "self_attn."),
            "norm2": PartSpec("rmsnorm", norm, p + "post_attention_layernorm."),
            "ffn": PartSpec("swiglu", dict(hidden_size=cfg.hidden_size,
                                           intermediate_size=cfg.intermediate_size), p + "mlp."),
        }))
    return ModelDescription(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size),
                           "model.embed_tokens."),
        layers=tuple(layers),
        order=tuple(ExecEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps), "model.norm."),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                                      tied=cfg.tie_word_embeddings), "lm_head."),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, describe_qwen3, model_types=("qwen3",))
