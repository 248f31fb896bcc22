"""Gemma 2 configuration: the keys of its config.json.

Defaults are those of gemma-2-2b, as in wlejon/brolm
(include/brolm/gemma2_config.h:27-43; parsed in src/gemma2_config.cpp:53-73).
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar

from .base import ConfigError, ModelConfig


@dataclasses.dataclass
class Gemma2Config(ModelConfig):
    architecture: ClassVar[str] = "Gemma2ForCausalLM"
    model_types: ClassVar[tuple[str, ...]] = ("gemma2",)

    vocab_size: int = 256000
    hidden_size: int = 2304
    intermediate_size: int = 9216
    num_hidden_layers: int = 26
    num_attention_heads: int = 8
    num_key_value_heads: int = 4
    head_dim: int = 256
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = True
    query_pre_attn_scalar: float = 256.0
    sliding_window: int = 4096
    attn_logit_softcapping: float = 50.0
    final_logit_softcapping: float = 30.0
    max_position_embeddings: int = 8192
    hidden_activation: str = "gelu_pytorch_tanh"
    layer_types: tuple = ()
    bos_token_id: int = 2
    eos_token_id: int = 1

    def validate(self) -> None:
        """Cross-field checks (src/gemma2_config.cpp:186-210).

        Unlike wlejon/brolm, ``query_pre_attn_scalar`` may differ from
        ``head_dim``: the score scale is taken from it directly.
        """
        who = "Gemma2Config"
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size", "head_dim"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{who}: config has non-positive dimension ({key}={getattr(self, key)})")
        if self.num_attention_heads <= 0 or self.num_key_value_heads <= 0:
            raise ConfigError(f"{who}: num_attention_heads / num_key_value_heads must be positive")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"{who}: num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"{who}: head_dim must be even (RoPE rotates dimension pairs)")
        if not self.query_pre_attn_scalar > 0:
            raise ConfigError(f"{who}: query_pre_attn_scalar must be positive")
        if self.sliding_window < 1:
            raise ConfigError(f"{who}: sliding_window must be at least 1")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"{who}: rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError(f"{who}: rope_theta must be positive")
        if self.attn_logit_softcapping < 0 or self.final_logit_softcapping < 0:
            raise ConfigError(f"{who}: soft-capping values must be >= 0 (0 switches one off)")
        if self.hidden_activation not in ("gelu_pytorch_tanh", "gelu_tanh"):
            raise ConfigError(f"{who}: hidden_activation '{self.hidden_activation}' is not gelu-tanh")
        if self.layer_types:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(f"{who}: layer_types has {len(self.layer_types)} entries for "
                                  f"{self.num_hidden_layers} layers")
            for kind in self.layer_types:
                if kind not in ("sliding_attention", "full_attention"):
                    raise ConfigError(f"{who}: unknown layer type '{kind}'")

    # derived sizes -------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def is_sliding(self, layer: int) -> bool:
        """Even layers slide, odd ones are global (src/gemma2.cpp:364), unless
        config.json lists ``layer_types``."""
        if self.layer_types:
            return self.layer_types[layer] == "sliding_attention"
        return layer % 2 == 0
