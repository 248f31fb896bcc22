"""The cache of a model: paged keys and values per layer, and fixed-size state.

Every live sequence holds one *slot*.  A slot records the sequence's length
and, for every group of layers, the pages that hold its keys and values.
Layers whose needs are equal form a *group* with storage of its own:

* a group that keeps all keys grows by one page every ``page_size`` tokens;
* a group that keeps a window of W keys holds a ring of
  ``round_up(W, page_size)`` places per sequence; position p lives at ring
  index ``p % ring``, so a sequence never holds more than ``ring/page_size``
  pages of it however long it grows;
* a state group holds one tensor of fixed shape per (layer, slot), zeroed when
  the slot is taken.

Storage of a key/value group is ``[layer][page][kv_head][page_size][head_dim]``
for keys and the same for values; all layers of a group share the page ids, so
one page table per group serves all of them.  Pages and slots go back to their
pools when a sequence ends and are handed out again.

wlejon/brolm keeps one sequence with a full-length store on every layer
(src/gemma2.cpp:239-251); slots, pages, the ring and the state group are this
framework's own design.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Sequence, Union

import torch

from .pages import CacheError, CacheFull, PagePool, SlotTable

PAGE_SIZE = 64


@dataclasses.dataclass(frozen=True)
class KVSpec:
    """Keys and values of ``n_kv`` heads of ``head_dim``; ``window`` None keeps all."""
    n_kv: int
    head_dim: int
    window: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class StateSpec:
    """A tensor of fixed ``shape`` per sequence (``dtype`` None: the cache's)."""
    shape: tuple
    dtype: Optional[torch.dtype] = None


CacheSpec = Union[KVSpec, StateSpec]


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class KVGroup:
    def __init__(self, spec: KVSpec, entries: list[int], num_pages: int, page_size: int, dtype, device):
        self.spec = spec
        self.entries = entries
        self.page_size = page_size
        self.ring = _round_up(spec.window, page_size) if spec.window else None
        self.pool = PagePool(num_pages)
        shape = (len(entries), num_pages, spec.n_kv, page_size, spec.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pages: dict[int, list[int]] = {}     # slot -> page ids in ring/position order

    @property
    def ring_tokens(self) -> int:
        """Ring length handed to the kernels; a group that keeps all keys never wraps."""
        return self.ring if self.ring else (1 << 30)

    def pages_for(self, length: int) -> int:
        held = length if self.ring is None else min(length, self.ring)
        return (held + self.page_size - 1) // self.page_size


class StateGroup:
    def __init__(self, spec: StateSpec, entries: list[int], num_slots: int, dtype, device):
        self.spec = spec
        self.entries = entries
        # one row more than there are slots: the padding rows of a captured decode step point there, so a
        # mixer that indexes its state with the step's slots never touches a live sequence's state for them
        self.data = torch.zeros((len(entries), num_slots + 1) + tuple(spec.shape), dtype=spec.dtype or dtype,
                                device=device)


@dataclasses.dataclass
class CacheEntry:
    """Where one schedule entry keeps its cache: a group and a layer index in it."""
    group: Union[KVGroup, StateGroup]
    group_id: int
    index: int

    @property
    def k(self) -> torch.Tensor:
        return self.group.k[self.index]

    @property
    def v(self) -> torch.Tensor:
        return self.group.v[self.index]

    @property
    def state(self) -> torch.Tensor:
        return self.group.data[self.index]


class Cache:
    """Slots, page pools and storage for the cache needs of a schedule.

    ``specs[i]`` is what schedule entry i keeps (None: nothing of its own).
    ``max_tokens`` is the most tokens live sequences hold at one time, each
    sequence's count rounded up to a multiple of the page size.
    """

    def __init__(self, specs: Sequence[Optional[CacheSpec]], max_tokens: int, dtype: torch.dtype,
                 device: Union[str, torch.device], page_size: int = PAGE_SIZE, max_slots: Optional[int] = None):
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        if page_size <= 0 or page_size % 32 != 0:
            raise CacheError("page_size must be a positive multiple of 32")
        self.page_size = page_size
        self.num_pages = (max_tokens + page_size - 1) // page_size
        self.max_tokens = self.num_pages * page_size
        self.max_slots = max_slots if max_slots is not None else min(self.num_pages, 1024)
        if self.max_slots <= 0:
            raise CacheError("max_slots must be positive")
        self.dtype, self.device = dtype, torch.device(device)
        self.slots = SlotTable(self.max_slots)
        self.padding_slot = self.max_slots        # the slot number of padding rows: a spare row of every state group
        self.lengths = [0] * self.max_slots
        self.epochs = [0] * self.max_slots        # how often a slot has been taken: tells one tenant from the next
        self.kv_groups: list[KVGroup] = []
        self.state_groups: list[StateGroup] = []
        self.entries: list[Optional[CacheEntry]] = [None] * len(specs)

        by_spec: dict[CacheSpec, list[int]] = {}
        for i, s in enumerate(specs):
            if s is not None:
                by_spec.setdefault(s, []).append(i)
        for spec, idxs in by_spec.items():
            if isinstance(spec, KVSpec):
                pages = self.num_pages
                if spec.window:
                    ring_pages = _round_up(spec.window, page_size) // page_size
                    pages = min(pages, self.max_slots * ring_pages)
                g = KVGroup(spec, idxs, pages, page_size, dtype, self.device)
                gid = len(self.kv_groups)
                self.kv_groups.append(g)
            elif isinstance(spec, StateSpec):
                g = StateGroup(spec, idxs, self.max_slots, dtype, self.device)
                gid = len(self.state_groups)
                self.state_groups.append(g)
            else:
                raise CacheError(f"unknown cache spec {spec!r}")
            for j, i in enumerate(idxs):
                self.entries[i] = CacheEntry(g, gid, j)

    # slots ----------------------------------------------------------------
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        self.epochs[slot] += 1
        for g in self.kv_groups:
            g.pages[slot] = []
        for g in self.state_groups:
            g.data[:, slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is given back but is not held")
        for g in self.kv_groups:
            g.pool.free(g.pages.pop(slot))
        self.lengths[slot] = 0
        self.slots.free(slot)

    def length(self, slot: int) -> int:
        self._check_slot(slot)
        return self.lengths[slot]

    def _check_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held")

    # growth ---------------------------------------------------------------
    def reserve(self, new_lengths: dict[int, int]) -> None:
        """Make room for every slot to grow to its new length; all or nothing."""
        need = [0] * len(self.kv_groups)
        for slot, n in new_lengths.items():
            self._check_slot(slot)
            if n < self.lengths[slot]:
                raise CacheError(f"slot {slot} cannot shrink from {self.lengths[slot]} to {n}")
            for gi, g in enumerate(self.kv_groups):
                need[gi] += max(0, g.pages_for(n) - len(g.pages[slot]))
        for gi, g in enumerate(self.kv_groups):
            if need[gi] > g.pool.free_pages:
                raise CacheFull(
                    f"the step needs {need[gi]} more pages of {g.page_size} tokens in the cache group of "
                    f"{g.spec} and {g.pool.free_pages} of {g.pool.num_pages} are free; "
                    f"the cache was sized for {self.max_tokens} tokens")
        for slot, n in new_lengths.items():
            for g in self.kv_groups:
                extra = g.pages_for(n) - len(g.pages[slot])
                if extra > 0:
                    g.pages[slot].extend(g.pool.alloc(extra))

    def commit(self, new_lengths: dict[int, int]) -> None:
        for slot, n in new_lengths.items():
            self.lengths[slot] = n

    # views ----------------------------------------------------------------
    def page_table(self, group_id: int, slots: Sequence[int], width: Optional[int] = None,
                   rows: Optional[int] = None) -> torch.Tensor:
        """Host int32 table [rows or len(slots), width] of the slots' pages; a
        negative slot (padding row) and unused places read as page 0."""
        import numpy as np
        g = self.kv_groups[group_id]
        lists = [g.pages[s] if s >= 0 else [] for s in slots]
        w = max([len(l) for l in lists] + [1])
        if width is not None:
            if width < w:
                raise CacheError("page table width is too small")
            w = width
        table = np.zeros((rows or len(slots), w), dtype=np.int32)
        for r, l in enumerate(lists):
            if l:
                table[r, :len(l)] = l
        return torch.from_numpy(table)

    def write_rows(self, group_id: int, slots: Sequence[int], old: Sequence[int], new: Sequence[int]):
        """Where each new token of a step goes in a group's storage: one int per
        token (sequences back to back), page * page_size + place, or -1 for a
        token the ring will not keep (a later token of the step takes its place)."""
        import numpy as np
        g = self.kv_groups[group_id]
        out = []
        for s, a, b in zip(slots, old, new):
            if s < 0:
                out.append(np.full(b - a, -1, dtype=np.int64))
                continue
            pos = np.arange(a, b, dtype=np.int64)
            ridx = pos % g.ring if g.ring else pos
            pages = np.asarray(g.pages[s], dtype=np.int64)
            rows = pages[ridx // g.page_size] * g.page_size + ridx % g.page_size
            if g.ring:
                rows[pos < b - g.ring] = -1
            out.append(rows)
        return np.concatenate(out) if out else np.zeros(0, dtype=np.int64)

    def pages_signature(self, group_id: int, slots: Sequence[int]) -> tuple:
        """Changes whenever the page table of these slots does: pages are only ever appended to a
        slot's list, and a slot that was given back and taken again has a new epoch."""
        g = self.kv_groups[group_id]
        return tuple((s, self.epochs[s], len(g.pages[s])) if s >= 0 else (-1, 0, 0) for s in slots)

    def decode_rows(self, group_id: int, slots: Sequence[int], positions: Sequence[int]) -> list:
        """``write_rows`` for one new token per slot at ``positions`` (the decode step), without arrays."""
        g = self.kv_groups[group_id]
        P, ring = g.page_size, g.ring
        out = []
        for s, pos in zip(slots, positions):
            if s < 0:
                out.append(-1)
                continue
            r = pos % ring if ring else pos
            out.append(g.pages[s][r // P] * P + r % P)
        return out

    def entry(self, i: int) -> CacheEntry:
        e = self.entries[i]
        if e is None:
            raise CacheError(f"schedule entry {i} keeps no cache")
        return e

    @property
    def live_slots(self) -> int:
        return self.max_slots - self.slots.free_slots

    def bytes(self) -> int:
        n = 0
        for g in self.kv_groups:
            n += g.k.numel() * g.k.element_size() * 2
        for g in self.state_groups:
            n += g.data.numel() * g.data.element_size()
        return n
