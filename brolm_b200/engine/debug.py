"""Checks of a step's description before it reaches the device (``BROLM_DEBUG=1``).

Every index that a kernel of this library follows into memory is written by
the host: token ids, positions, lengths, page tables, the places of the new
keys and values in the cache, the rows whose logits are wanted, the slots.  A
wrong one would read or write someone else's pages, or fault the GPU.  With
``BROLM_DEBUG=1`` in the environment every step's arrays are checked against
the cache's own bookkeeping before they are copied to the device, and a step
that fails raises ``StepError`` without launching anything.  The checks cost a
few passes over arrays of the step's size; they are off by default.
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import numpy as np

ENABLED = os.environ.get("BROLM_DEBUG", "0") not in ("", "0")


class StepCheckError(ValueError):
    pass


def check_step(cache, mode: str, vocab: int, tokens: Optional[np.ndarray], slots: Sequence[int], positions: np.ndarray,
               tok_seq: np.ndarray, kv_len: np.ndarray, page_tables: Sequence[np.ndarray],
               cache_rows: Sequence[np.ndarray], wanted: Optional[np.ndarray]) -> None:
    """Raise ``StepCheckError`` naming the first array and index that is out of bounds or inconsistent.

    ``slots``: the slot of each row, negative or ``cache.padding_slot`` for padding rows;
    ``positions`` / ``tok_seq`` / ``cache_rows[g]``: one entry per token of the step, padding included;
    ``kv_len``: one entry per row; ``page_tables[g]``: [rows, width]; ``wanted``: token indices."""
    def fail(what: str):
        raise StepCheckError(f"debug: {what}")

    n_tokens, rows = len(positions), len(kv_len)
    live_row = np.array([0 <= s < cache.max_slots for s in slots] + [False] * (rows - len(slots)))
    if tokens is not None and len(tokens) and (tokens.min() < 0 or tokens.max() >= vocab):
        fail(f"token id outside [0, {vocab}) at token {int(np.argmax((tokens < 0) | (tokens >= vocab)))}")
    if len(tok_seq) != n_tokens or (n_tokens and (tok_seq.min() < 0 or tok_seq.max() >= rows)):
        fail("tok_seq names a row that the step does not have")
    live_tok = live_row[tok_seq] if n_tokens else np.zeros(0, dtype=bool)
    if np.any(positions[~live_tok] != -1):
        fail("a padding row's token has a position")
    if np.any((positions[live_tok] < 0) | (positions[live_tok] >= cache.max_positions)):
        bad = int(np.flatnonzero(live_tok)[np.argmax((positions[live_tok] < 0) | (positions[live_tok] >= cache.max_positions))])
        fail(f"position {int(positions[bad])} of token {bad} is outside [0, {cache.max_positions})")
    if np.any(kv_len[~live_row] != 0):
        fail("a padding row has a length")
    for r in np.flatnonzero(live_row):
        s = slots[r]
        if not cache.slots.is_held(s):
            fail(f"row {r} names slot {s}, which no sequence holds")
        mine = positions[tok_seq == r]
        if len(mine) == 0 or int(kv_len[r]) != int(mine.max()) + 1:
            fail(f"row {r}: length {int(kv_len[r])} is not its last position + 1")
        if mode == "decode" and len(mine) != 1:
            fail(f"row {r} of a decode step brings {len(mine)} tokens")
    held = [s for r, s in enumerate(slots) if live_row[r]]
    if len(set(held)) != len(held):
        fail("a slot is named by two rows")
    if wanted is not None and len(wanted) and (wanted.min() < 0 or wanted.max() >= n_tokens):
        fail(f"a wanted row is outside the step's {n_tokens} tokens")
    for g, (grp, table, crow) in enumerate(zip(cache.kv_groups, page_tables, cache_rows)):
        P, pool_pages = grp.page_size, grp.pool.num_pages
        if table.shape[0] < rows and table.shape[0] < len(slots):
            fail(f"group {g}: the page table has fewer rows than the step")
        if table.size and (table.min() < 0 or table.max() >= pool_pages):
            fail(f"group {g}: a page table entry is outside the pool of {pool_pages} pages")
        seen: dict[int, int] = {}
        for r in np.flatnonzero(live_row):
            keys = int(kv_len[r]) if not grp.ring else min(int(kv_len[r]), grp.ring)
            need = (keys + P - 1) // P
            if need > table.shape[1]:
                fail(f"group {g}, row {r}: {need} pages are needed and the table is {table.shape[1]} wide")
            own = cache.kv_groups[g].pages[slots[r]]
            if list(table[r, :need]) != list(own[:need]):
                fail(f"group {g}, row {r}: the page table differs from the pages slot {slots[r]} holds")
            for p in own:
                if seen.setdefault(int(p), r) != r:
                    fail(f"group {g}: page {int(p)} belongs to rows {seen[int(p)]} and {r}")
        if len(crow) != n_tokens:
            fail(f"group {g}: {len(crow)} cache rows for {n_tokens} tokens")
        if np.any(crow[~live_tok] != -1):
            fail(f"group {g}: a padding row's token has a place in the cache")
        kept = live_tok & (crow >= 0)
        if np.any(crow[kept] >= pool_pages * P):
            fail(f"group {g}: a cache row is outside the pool")
        if len(np.unique(crow[kept])) != int(kept.sum()):
            fail(f"group {g}: two tokens of the step go to one place in the cache")
        for t in np.flatnonzero(kept):
            r = int(tok_seq[t])
            pos = int(positions[t])
            place = pos % grp.ring if grp.ring else pos
            want = cache.kv_groups[g].pages[slots[r]][place // P] * P + place % P
            if int(crow[t]) != want:
                fail(f"group {g}, token {t}: cache row {int(crow[t])}, but position {pos} of slot {slots[r]} lives at {want}")
        # a token that is not kept must be one that a later token of the same step overwrites in the ring
        for t in np.flatnonzero(live_tok & (crow < 0)):
            r = int(tok_seq[t])
            if not grp.ring or int(positions[t]) + grp.ring >= int(kv_len[r]):
                fail(f"group {g}, token {t}: not kept, although nothing of this step takes its place")
