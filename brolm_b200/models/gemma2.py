"""Gemma 2 as a layout of parts (wlejon/brolm src/gemma2.cpp:143-235 for the
tensor names, :326-415 for the order of operations).

Per layer: attention with rotary positions, score scale
``query_pre_attn_scalar ** -0.5``, tanh soft-capping and, on sliding layers, a
window; a gated gelu-tanh feed-forward; four RMSNorms with gain ``1 + w``.
The embedding is scaled by sqrt(hidden); the output matrix is the embedding
when the checkpoint has no ``lm_head.weight``; the logits are soft-capped.
"""
from __future__ import annotations

import math

from ..config import Gemma2Config, register_architecture
from ..parts import BlockSpec, EmbeddingSpec, HeadSpec, LayerCall, ModelLayout, PartSpec


def gemma2_layout(cfg: Gemma2Config) -> ModelLayout:
    H = cfg.hidden_size

    def norm(name: str) -> PartSpec:
        return PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.rms_norm_eps, offset=1.0), {"weight": name})

    rope = PartSpec("position", "rope", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta))
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec(
            "mixer", "attention",
            dict(hidden=H, n_q=cfg.num_attention_heads, n_kv=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                 scale=float(cfg.query_pre_attn_scalar) ** -0.5, softcap=cfg.attn_logit_softcapping,
                 window=cfg.sliding_window if cfg.is_sliding(i) else None, position=rope),
            {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
             "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"})
        ffn = PartSpec(
            "feedforward", "gated", dict(hidden=H, inter=cfg.intermediate_size, activation="gelu_tanh"),
            {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight", "down": p + "mlp.down_proj.weight"})
        blocks.append(BlockSpec(
            mixer=mixer, feedforward=ffn,
            pre_mixer_norm=norm(p + "input_layernorm.weight"),
            post_mixer_norm=norm(p + "post_attention_layernorm.weight"),
            pre_ffn_norm=norm(p + "pre_feedforward_layernorm.weight"),
            post_ffn_norm=norm(p + "post_feedforward_layernorm.weight")))
    return ModelLayout(
        embedding=EmbeddingSpec("model.embed_tokens.weight", cfg.vocab_size, H,
                                scale=float(math.sqrt(H))),
        blocks=blocks,
        schedule=[LayerCall(i) for i in range(cfg.num_hidden_layers)],
        final_norm=norm("model.norm.weight"),
        head=HeadSpec("lm_head.weight",
                      tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None,
                      softcap=cfg.final_logit_softcapping),
        optional_prefix="model.",
        max_positions=cfg.max_position_embeddings)


register_architecture(Gemma2Config, gemma2_layout)
