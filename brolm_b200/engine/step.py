"""The step function: a batch of sequences through the model, from the cache.

A step either starts all of its sequences (every slot is empty; the prompts,
of unequal lengths, run packed back to back) or extends each of them by one
token.  It runs only the tokens it is given, reads what earlier steps left in
the cache, and returns float32 logits at the wanted places.

wlejon/brolm's forward/forward_last take one sequence at ``cache_len``
(include/brolm/gemma2.h:119-129); the batched form is this framework's own.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import Cache, CacheError
from .context import StepContext
from .model import DecoderModel


class StepError(ValueError):
    pass


class Engine:
    """A model with a cache: slots, steps, and nothing else."""

    def __init__(self, model: DecoderModel, max_tokens: int, max_slots: Optional[int] = None,
                 max_seq_len: Optional[int] = None):
        self.model = model
        self.cache: Cache = model.new_cache(max_tokens, max_slots, max_seq_len)
        self.device = model.device
        self.vocab = model.layout.embedding.vocab

    # slots ----------------------------------------------------------------
    def open(self, n: int = 1) -> list[int]:
        """Take n empty slots (all or none)."""
        if n > self.cache.slots.free_slots:
            raise CacheError(f"{n} sequences asked for, {self.cache.slots.free_slots} slots free")
        return [self.cache.alloc_slot() for _ in range(n)]

    def close(self, slots: Sequence[int]) -> None:
        for s in slots:
            self.cache.free_slot(s)

    # the step -------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Run ``tokens[i]`` on ``slots[i]``; return logits [wanted, vocab] (float32, device).

        ``want[i]`` lists the places among ``tokens[i]`` whose logits are
        wanted (default: the last one of each), in the order given.
        """
        ctx, tok_dev, rows = self._prepare(slots, tokens, want)
        logits = self.model.forward(ctx, tok_dev, rows)
        self.cache.commit(dict(zip(slots, ctx.host_lengths)))
        return logits

    def _prepare(self, slots, tokens, want):
        B = len(slots)
        if B == 0 or len(tokens) != B:
            raise StepError("step: needs as many token lists as slots, and at least one")
        if len(set(slots)) != B:
            raise StepError("step: a slot is named twice")
        cache = self.cache
        old = [cache.length(s) for s in slots]
        n_new = [len(t) for t in tokens]
        if min(n_new) <= 0:
            raise StepError("step: every sequence must bring at least one token")
        if all(o == 0 for o in old):
            mode = "prefill"
        elif all(n == 1 for n in n_new) and all(o > 0 for o in old):
            mode = "decode"
        else:
            raise StepError("step: the sequences of a step must either all start at their first token "
                            "or all go on by one token")
        new_len = [o + n for o, n in zip(old, n_new)]
        if max(new_len) > cache.max_positions:
            raise StepError(f"step: a sequence would reach {max(new_len)} tokens; the cache was made for "
                            f"sequences of up to {cache.max_positions}")
        flat = np.fromiter((t for seq in tokens for t in seq), dtype=np.int64, count=sum(n_new))
        if flat.min() < 0 or flat.max() >= self.vocab:
            raise StepError(f"step: token id out of range [0, {self.vocab})")
        if want is None:
            want = [[n - 1] for n in n_new]
        if len(want) != B:
            raise StepError("step: 'want' needs one list per sequence")
        cache.reserve(dict(zip(slots, new_len)))

        T = int(sum(n_new))
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(n_new, out=cu[1:])
        rows = []
        for i, w in enumerate(want):
            for p in w:
                if not 0 <= p < n_new[i]:
                    raise StepError(f"step: wanted place {p} is outside the {n_new[i]} tokens given")
                rows.append(cu[i] + p)
        positions = np.concatenate([np.arange(o, o + n) for o, n in zip(old, n_new)])
        tok_seq = np.repeat(np.arange(B), n_new)
        tables = [cache.page_table(g, slots).numpy() for g in range(len(cache.kv_groups))]

        # one host buffer, one copy
        parts = [flat, positions, tok_seq, cu, np.asarray(new_len), np.asarray(slots), np.asarray(rows, dtype=np.int64)]
        parts += [t.reshape(-1) for t in tables]
        sizes = [p.size for p in parts]
        offs = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])])
        host = torch.zeros(int(offs[-1]), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        hv = host.numpy()
        for p, o in zip(parts, offs[:-1]):
            hv[o:o + p.size] = p
        dev = host.to(self.device, non_blocking=True)
        seg = [dev[int(o):int(o) + s] for o, s in zip(offs[:-1], sizes)]
        page_tables = [seg[7 + g].view(B, tables[g].shape[1]) for g in range(len(tables))]
        ctx = StepContext(mode=mode, dtype=self.model.dtype, device=self.device, cache=cache, batch=B, n_tokens=T,
                          slots=list(slots), positions=seg[1], tok_seq=seg[2], cu_q=seg[3], kv_len=seg[4],
                          slots_dev=seg[5], max_q_len=int(max(n_new)), page_tables=page_tables,
                          host_lengths=new_len)
        return ctx, seg[0], seg[6]
