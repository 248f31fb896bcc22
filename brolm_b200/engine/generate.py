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
    device = getattr(engine, "device", None)
    ahead = (hasattr(engine, "step_from") and isinstance(device, torch.device) and device.type == "cuda"
             and isinstance(sampler, Sampler))
    run = _run_batch_ahead if ahead else _run_batch
    for batch in batches:
        slots = engine.open(len(batch))
        try:
            run(engine, sampler, prompts, batch, slots, opts.max_new_tokens, stops, results, on_step)
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


def _run_batch_ahead(engine, sampler, prompts, batch, slots, max_new, stops, results, on_step) -> None:
    """``_run_batch`` for an engine on a GPU, one step ahead of the host.

    The ids a step draws stay on the device and feed the next step directly (``Engine.step_from``), so
    that step is queued before the host has read them; the host reads them on a second stream while
    the GPU is already busy, and learns one step late that a sequence has drawn a stop token.  The
    step that was queued for that sequence in the meantime is wasted (its row is sampled and thrown
    away, its slot goes back with the batch); what is returned, the random numbers of the draws and
    the budget are those of ``_run_batch``.
    """
    device = engine.device
    n = len(batch)
    side = torch.cuda.Stream(device=device)
    drawn_host = torch.empty(n, dtype=torch.int32, pin_memory=True)
    drawn_ready, ids_ready = torch.cuda.Event(), torch.cuda.Event()
    stopped = [False] * n
    queued = [0] * n                                   # tokens drawn or being drawn for each request
    rows = list(range(n))                              # the requests whose logits the last step left, in row order
    logits = engine.step([slots[a] for a in rows], [list(prompts[batch[a]]) for a in rows])
    streams, streams_of = None, None
    produced = 0
    while rows:
        if streams_of != rows:
            streams = torch.tensor([batch[a] for a in rows], dtype=torch.int32).to(device)
            streams_of = list(rows)
        ids = sampler(logits, streams, produced)
        produced += 1
        for a in rows:
            queued[a] += 1
        # the host's copy of the ids, on a stream of its own: the next step does not wait for it
        ids_ready.record()
        side.wait_event(ids_ready)
        with torch.cuda.stream(side):
            drawn_host[:len(rows)].copy_(ids, non_blocking=True)
            drawn_ready.record()
        ahead = [a for a in rows if not stopped[a] and queued[a] < max_new]
        if ahead:
            logits = engine.step_from([slots[a] for a in ahead], ids, [rows.index(a) for a in ahead])
        drawn_ready.synchronize()
        drawn = drawn_host[:len(rows)].tolist()
        if on_step:
            on_step(produced, len(rows))
        for a, tok in zip(rows, drawn):
            if stopped[a]:
                continue                                  # drawn for a sequence that had already ended
            if tok in stops:
                stopped[a] = True                         # the stop token is not returned
            else:
                results[batch[a]].append(int(tok))
        rows = ahead
