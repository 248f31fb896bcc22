"""The generation loop above the step function.

wlejon/brolm generates one sequence at a time
(include/brolm/detail/generate.h:78-123): prefill, sample, then one token per
step until eos or the budget.  This loop does the same for batches of
requests with unequal prompts: one prefill step for the whole batch, then one
decode step per token for the sequences still running.  A sequence that draws
a stop token leaves the batch (the stop token is not returned, generate.h:
106-118); its slot goes back with the others when the batch ends, and the
next batch uses the slots again.  An empty prompt or a budget <= 0 gives an
empty result (generate.h:87-89).
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch

from ..sampling import GenerateOptions, Sampler


def round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def plan_batches(lengths: Sequence[int], max_new: int, max_tokens: int, max_slots: int, page_size: int,
                 batch_size: Optional[int] = None) -> list[list[int]]:
    """Cut the requests, in order, into batches the cache can hold.

    A request counts as its prompt plus its budget, rounded up to whole pages.
    Requests with nothing to do (empty prompt) are left out of every batch.
    """
    batches: list[list[int]] = []
    cur: list[int] = []
    held = 0
    limit = min(max_slots, batch_size) if batch_size else max_slots
    for i, n in enumerate(lengths):
        if n <= 0 or max_new <= 0:
            continue
        need = round_up(n + max_new, page_size)
        if need > max_tokens:
            raise ValueError(f"request {i} needs {need} cache tokens; the cache holds {max_tokens}")
        if cur and (held + need > max_tokens or len(cur) >= limit):
            batches.append(cur)
            cur, held = [], 0
        cur.append(i)
        held += need
    if cur:
        batches.append(cur)
    return batches


def generate(engine, prompts: Sequence[Sequence[int]], eos_id: int = -1,
             opts: Optional[GenerateOptions] = None, batch_size: Optional[int] = None,
             sampler: Optional[Callable] = None,
             on_step: Optional[Callable[[int, int], None]] = None) -> list[list[int]]:
    """Generate for every prompt; returns only the new ids of each.

    ``engine`` offers ``open``, ``close``, ``step`` and a ``cache`` with
    ``max_tokens``, ``max_slots`` and ``page_size`` (``Engine`` does).
    ``sampler(logits, streams, counter) -> ids`` defaults to the device
    sampler for ``opts.sampling``.
    """
    opts = opts or GenerateOptions()
    sampler = sampler or Sampler(opts.sampling)
    stops = set(int(s) for s in opts.stop_ids if int(s) >= 0)
    if opts.stop_on_eos and eos_id is not None and eos_id >= 0:
        stops.add(int(eos_id))
    results: list[list[int]] = [[] for _ in prompts]
    cache = engine.cache
    batches = plan_batches([len(p) for p in prompts], opts.max_new_tokens, cache.max_tokens, cache.max_slots,
                           cache.page_size, batch_size)
    for batch in batches:
        slots = engine.open(len(batch))
        try:
            _run_batch(engine, sampler, prompts, batch, slots, opts.max_new_tokens, stops, results, on_step)
        finally:
            engine.close(slots)
    return results


def _run_batch(engine, sampler, prompts, batch, slots, max_new, stops, results, on_step) -> None:
    device = getattr(engine, "device", "cpu")
    active = list(range(len(batch)))                     # indices into batch / slots
    tokens = [list(prompts[r]) for r in batch]
    produced = 0
    streams, streams_of = None, None
    while active:
        logits = engine.step([slots[a] for a in active], [tokens[a] for a in active])
        if streams_of != active:                           # the request numbers change only when a request ends
            streams = torch.tensor([batch[a] for a in active], dtype=torch.int32).to(device)
            streams_of = list(active)
        drawn = sampler(logits, streams, produced).tolist()
        produced += 1
        if on_step:
            on_step(produced, len(active))
        still = []
        for a, tok in zip(active, drawn):
            if tok in stops:
                continue                                  # finished; the stop token is not returned
            results[batch[a]].append(int(tok))
            if len(results[batch[a]]) < max_new:
                tokens[a] = [int(tok)]
                still.append(a)
        active = still
