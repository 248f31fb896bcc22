"""What a step hands to the parts: who is in the batch and where their cache is."""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..cache import Cache, CacheEntry, KVGroup


@dataclasses.dataclass
class StepContext:
    """One step's batch as the parts see it.

    ``prefill`` steps start every sequence at position 0 with all of its
    tokens packed back to back; ``decode`` steps bring one token per sequence.
    Rows beyond the real sequences are padding: their position is -1, their
    ``kv_len`` is 0 and their slot is ``cache.padding_slot``, a spare row of
    every state group that belongs to no sequence; no kernel reads or writes
    keys and values for them.
    """
    mode: str                      # "prefill" | "decode"
    dtype: torch.dtype             # element type of activations and of the cache
    device: torch.device
    cache: Cache
    batch: int                     # rows, padding included
    n_tokens: int                  # packed tokens, padding included
    slots: list                    # host: slot of each row, -1 for padding
    positions: torch.Tensor        # int32 [n_tokens], -1 for padding
    tok_seq: torch.Tensor          # int32 [n_tokens], batch row of each token
    cu_q: torch.Tensor             # int32 [batch + 1]
    kv_len: torch.Tensor           # int32 [batch], length after this step
    slots_dev: torch.Tensor        # int32 [batch]
    max_q_len: int
    page_tables: list              # per key/value group: int32 [batch, width] on the device
    cache_rows: list               # per key/value group: int32 [n_tokens], page * page_size + place, or -1
    host_lengths: list             # host copy of kv_len
    max_kv_len: int = 0            # an upper bound of kv_len for sizing launches (a captured graph fixes it)
    ragged: bool = False           # decode: the lengths are far from equal (a hint for how attention cuts its work)

    def __post_init__(self):
        if not self.max_kv_len:
            self.max_kv_len = max(self.host_lengths) if self.host_lengths else 0

    def kv(self, entry: CacheEntry):
        """(k_pages, v_pages, page_table, ring, page_size) of a key/value entry."""
        g: KVGroup = entry.group
        return entry.k, entry.v, self.page_tables[entry.group_id], g.ring_tokens, g.page_size

    def state(self, entry: CacheEntry) -> torch.Tensor:
        """[max_slots + 1, *shape] state tensor of a state entry; index it with ``slots_dev``
        (the last row is the padding rows' own)."""
        return entry.state
