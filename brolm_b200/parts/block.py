"""Blocks: how a layer's parts are arranged around the residual stream.

An arrangement is a registered part of kind ``block`` like any other; a
layout names it in ``BlockSpec.kind``.  The one Gemma 2 needs is
``sandwich``:

    x = pre_mixer(h);  h += post_mixer(mixer(x))      (post_mixer may be absent)
    x = pre_ffn(h);    h += post_ffn(ffn(x))          (post_ffn, or the whole second line, may be absent)

Gemma 2 has all four norms (wlejon/brolm src/gemma2.cpp:345-387); a block
without the post norms is the usual pre-norm arrangement.  h is the float32
residual stream.  Each sum is fused with the norm before it and the norm after
it (the next block's entry norm included), so the residual stream is read
and written once per half block.

What the generic model asks of an arrangement:

* ``__init__(**parts)``: the built parts under the names the ``BlockSpec`` gave them;
* ``parts()``: name -> part (or None), for tensor names and the graph-safety check;
* ``entry_norm``: the norm that makes the block's input from the residual stream, or None
  when the block reads the stream itself (the block before fuses this norm with its last sum);
* ``cache_spec()``: what the block keeps per sequence between steps (its mixer's);
* ``forward(h, x, ctx, entry, writes_cache, next_norm)``: update ``h`` in place, ``x`` being
  ``entry_norm(h)``; return ``next_norm(h)`` when ``next_norm`` is given.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from .base import Part, PartSpec, register_part
from .norm import add_then_norm


@dataclasses.dataclass
class BlockSpec:
    """A block as a layout writes it down.  The six named fields are the parts of the
    ``sandwich`` arrangement; another arrangement may name further parts in ``more``."""
    mixer: Optional[PartSpec] = None
    feedforward: Optional[PartSpec] = None
    pre_mixer_norm: Optional[PartSpec] = None
    pre_ffn_norm: Optional[PartSpec] = None
    post_mixer_norm: Optional[PartSpec] = None
    post_ffn_norm: Optional[PartSpec] = None
    kind: str = "sandwich"
    more: dict = dataclasses.field(default_factory=dict)       # name -> PartSpec

    def part_specs(self) -> dict[str, PartSpec]:
        named = {f: getattr(self, f) for f in ("mixer", "feedforward", "pre_mixer_norm", "pre_ffn_norm",
                                               "post_mixer_norm", "post_ffn_norm")}
        named.update(self.more)
        return {k: v for k, v in named.items() if v is not None}


class Block(Part):
    kind = "block"

    def __init__(self, mixer: Part, feedforward: Optional[Part] = None, pre_mixer_norm: Optional[Part] = None,
                 pre_ffn_norm: Optional[Part] = None, post_mixer_norm: Optional[Part] = None,
                 post_ffn_norm: Optional[Part] = None):
        if pre_mixer_norm is None:
            raise ValueError("block: the sandwich arrangement needs a norm before its mixer")
        if (feedforward is None) != (pre_ffn_norm is None):
            raise ValueError("block: a feed-forward and its pre-norm come together")
        self.mixer, self.feedforward = mixer, feedforward
        self.pre_mixer_norm, self.pre_ffn_norm = pre_mixer_norm, pre_ffn_norm
        self.post_mixer_norm, self.post_ffn_norm = post_mixer_norm, post_ffn_norm

    def parts(self) -> dict[str, Optional[Part]]:
        return {"mixer": self.mixer, "feedforward": self.feedforward, "pre_mixer_norm": self.pre_mixer_norm,
                "pre_ffn_norm": self.pre_ffn_norm, "post_mixer_norm": self.post_mixer_norm,
                "post_ffn_norm": self.post_ffn_norm}

    @property
    def entry_norm(self) -> Optional[Part]:
        return self.pre_mixer_norm

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, h: torch.Tensor, x: torch.Tensor, ctx, entry, writes_cache: bool,
                next_norm: Optional[Part]) -> Optional[torch.Tensor]:
        """h: residual stream (updated in place); x = pre_mixer_norm(h).
        Returns next_norm(h) for the block that follows, if there is one."""
        y = self.mixer.forward(x, ctx, entry, writes_cache)
        if self.feedforward is None:
            return add_then_norm(h, y, self.post_mixer_norm, next_norm, ctx.dtype)
        x = add_then_norm(h, y, self.post_mixer_norm, self.pre_ffn_norm, ctx.dtype)
        y = self.feedforward.forward(x, ctx)
        return add_then_norm(h, y, self.post_ffn_norm, next_norm, ctx.dtype)


register_part("block", "sandwich", Block)
