"""A block: one mixer and one feed-forward with the norms around them.

    x = pre_mixer(h);  h += post_mixer(mixer(x))      (post_mixer may be absent)
    x = pre_ffn(h);    h += post_ffn(ffn(x))          (post_ffn may be absent)

Gemma 2 has all four norms (wlejon/brolm src/gemma2.cpp:345-387); a block
without the post norms is the usual pre-norm arrangement.  h is the float32
residual stream.  Each sum is fused with the norm before it and the norm after
it (the next block's pre_mixer norm included), so the residual stream is read
and written once per half block.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from .base import Part, PartSpec
from .norm import add_then_norm


@dataclasses.dataclass
class BlockSpec:
    mixer: PartSpec
    feedforward: PartSpec
    pre_mixer_norm: PartSpec
    pre_ffn_norm: PartSpec
    post_mixer_norm: Optional[PartSpec] = None
    post_ffn_norm: Optional[PartSpec] = None


class Block:
    def __init__(self, mixer: Part, feedforward: Part, pre_mixer_norm: Part, pre_ffn_norm: Part,
                 post_mixer_norm: Optional[Part] = None, post_ffn_norm: Optional[Part] = None):
        self.mixer, self.feedforward = mixer, feedforward
        self.pre_mixer_norm, self.pre_ffn_norm = pre_mixer_norm, pre_ffn_norm
        self.post_mixer_norm, self.post_ffn_norm = post_mixer_norm, post_ffn_norm

    def parts(self) -> dict[str, Optional[Part]]:
        return {"mixer": self.mixer, "feedforward": self.feedforward, "pre_mixer_norm": self.pre_mixer_norm,
                "pre_ffn_norm": self.pre_ffn_norm, "post_mixer_norm": self.post_mixer_norm,
                "post_ffn_norm": self.post_ffn_norm}

    def forward(self, h: torch.Tensor, x: torch.Tensor, ctx, entry, writes_cache: bool,
                next_norm: Optional[Part]) -> Optional[torch.Tensor]:
        """h: residual stream (updated in place); x = pre_mixer_norm(h).
        Returns next_norm(h) for the block that follows, if there is one."""
        y = self.mixer.forward(x, ctx, entry, writes_cache)
        x = add_then_norm(h, y, self.post_mixer_norm, self.pre_ffn_norm, ctx.dtype)
        y = self.feedforward.forward(x, ctx)
        return add_then_norm(h, y, self.post_ffn_norm, next_norm, ctx.dtype)
