"""A model written down as data: which parts, in which order, under which
tensor names.  An architecture is one function from its configuration to a
``ModelLayout``; the generic model in ``engine/model.py`` builds and runs it.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

from .base import PartSpec
from .block import BlockSpec


@dataclasses.dataclass
class LayerCall:
    """One entry of the schedule: run ``block``.  ``cache_of`` None: the call
    keeps a cache of its own.  ``cache_of`` = j: it reads the cache that
    schedule entry j wrote in this step and writes none."""
    block: int
    cache_of: Optional[int] = None


@dataclasses.dataclass
class EmbeddingSpec:
    tensor: str            # checkpoint name, (vocab, hidden)
    vocab: int
    hidden: int
    scale: float = 1.0     # multiplies the looked-up row, in float32


@dataclasses.dataclass
class HeadSpec:
    tensor: str                       # checkpoint name of the output matrix, (vocab, hidden)
    tied_to: Optional[str] = None     # used when ``tensor`` is absent from the checkpoint
    softcap: float = 0.0              # cap * tanh(logits / cap); 0 switches it off


@dataclasses.dataclass
class ModelLayout:
    embedding: EmbeddingSpec
    blocks: list                      # list[BlockSpec]
    schedule: list                    # list[LayerCall]
    final_norm: PartSpec
    head: HeadSpec
    optional_prefix: str = ""         # a checkpoint may carry all names without this prefix
    max_positions: int = 0            # the architecture's own limit, 0: none
    weight_std: float = 0.02          # random-weights mode: matrices and tables
    norm_std: float = 0.1             # random-weights mode: vectors

    def __post_init__(self):
        for i, call in enumerate(self.schedule):
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"schedule entry {i} names block {call.block} of {len(self.blocks)}")
            if call.cache_of is not None:
                j = call.cache_of
                if not 0 <= j < i or self.schedule[j].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {j}, which must come "
                                     f"earlier and own its cache")
