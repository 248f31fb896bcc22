"""The step function: a batch of sequences through the model, from the cache.

A step either starts all of its sequences (every slot is empty; the prompts,
of unequal lengths, run packed back to back) or extends each of them by one
token.  It runs only the tokens it is given, reads what earlier steps left in
the cache, and returns float32 logits at the wanted places.

Decode steps are replayed from a captured CUDA graph: the step's tokens,
positions, lengths and page tables live in a device buffer of fixed layout
that one host-to-device copy refreshes, so the ~300 launches of a step cost
one graph launch (the idea of device-resident step state is wlejon/brolm's,
src/detail/dense_decoder.cpp:335-524, which it does not wire for Gemma 2,
include/brolm/gemma2.h:42-43).  A batch is padded to the next power of two;
padding rows have position -1 and length 0 and change no result.

wlejon/brolm's forward/forward_last take one sequence at ``cache_len``
(include/brolm/gemma2.h:119-129); the batched form is this framework's own.
"""
from __future__ import annotations

import dataclasses
import gc
from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache import Cache, CacheError
from . import debug
from .context import StepContext
from .model import DecoderModel


class StepError(ValueError):
    pass


@dataclasses.dataclass
class _Plan:
    mode: str
    slots: list
    n_new: list
    old: list
    new_len: list
    flat: np.ndarray        # all tokens of the step, packed
    rows: list              # packed row of every wanted place


def _next_pow2(n: int) -> int:
    return 1 << max(0, (n - 1).bit_length())


def _checked(*args) -> None:
    """The step's arrays against the cache's bookkeeping (``BROLM_DEBUG=1``); nothing is launched if they fail."""
    try:
        debug.check_step(*args)
    except debug.StepCheckError as e:
        raise StepError(str(e)) from None


def _ragged(lengths: Sequence[int]) -> bool:
    """Whether the longest sequence of a decode step is well beyond the mean (by a quarter)."""
    return len(lengths) > 1 and max(lengths) * len(lengths) > 1.25 * sum(lengths)


class _DecodeGraph:
    """One captured decode step for a padded batch size and a bound on the lengths."""

    def __init__(self, engine: "Engine", rows: int, kv_cap: int, ragged: bool = False):
        cache, dev = engine.cache, engine.device
        self.rows, self.kv_cap = rows, kv_cap
        self.widths = []
        for g in cache.kv_groups:
            w = (cache.max_positions + g.page_size - 1) // g.page_size
            if g.ring:
                w = min(w, g.ring // g.page_size)
            self.widths.append(max(1, w))
        n = 4 * rows + sum(rows * w for w in self.widths) + rows * len(self.widths)
        self.pick_off = n                    # last: which element of a tensor of drawn ids each row's token is
        n += rows
        self.host = torch.zeros(n, dtype=torch.int32, pin_memory=True)
        self.hv = self.host.numpy()
        self.table_sig = [None] * len(self.widths)      # what the page tables in the pinned buffer were made from
        self.dev = torch.zeros(n, dtype=torch.int32, device=dev)
        seg = [self.dev[i * rows:(i + 1) * rows] for i in range(4)]
        off = 4 * rows
        tables = []
        for w in self.widths:
            tables.append(self.dev[off:off + rows * w].view(rows, w))
            off += rows * w
        self.rows_off = off
        cache_rows = [self.dev[off + g * rows:off + (g + 1) * rows] for g in range(len(self.widths))]
        self.tokens = seg[0]
        self.pick = self.dev[self.pick_off:self.pick_off + rows]
        ar = torch.arange(rows + 1, dtype=torch.int32, device=dev)
        self.ctx = StepContext(
            mode="decode", dtype=engine.model.dtype, device=dev, cache=cache, batch=rows, n_tokens=rows, slots=[],
            positions=seg[1], tok_seq=ar[:rows].clone(), cu_q=ar, kv_len=seg[2], slots_dev=seg[3], max_q_len=1,
            page_tables=tables, cache_rows=cache_rows, host_lengths=[], max_kv_len=kv_cap, ragged=ragged)
        self.all_rows = ar[:rows].clone()
        # an all-padding state: the warm-up pass touches no cache
        self.hv[:] = 0
        self.hv[rows:2 * rows] = -1
        self.hv[3 * rows:4 * rows] = cache.padding_slot
        self.hv[self.rows_off:self.pick_off] = -1
        self.dev.copy_(self.host)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            engine.model.forward(self.ctx, self.tokens, self.all_rows)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.copied = torch.cuda.Event()
        self.copied.record()
        self.graph = torch.cuda.CUDAGraph()
        before = kernels.launch_count()
        # Nothing may free device memory while the stream is capturing: objects that the collector
        # would destroy in the middle of it (an older engine with graphs of its own) are collected now,
        # and the collector stays off until the capture has ended.
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, pool=engine._graph_pool):
                self.logits = engine.model.forward(self.ctx, self.tokens, self.all_rows)
                self.hidden = engine.model.last_hidden
        finally:
            if was_enabled:
                gc.enable()
        self.kernels = kernels.launch_count() - before      # this library's kernels in one replay

    def run(self, plan: _Plan, cache: Cache, ids: Optional[torch.Tensor] = None,
            pick: Optional[Sequence[int]] = None) -> torch.Tensor:
        """``ids``/``pick``: the tokens are not the plan's but ``ids[pick[i]]``, ids an int32 tensor on the
        device (what a sampler has just drawn): they are gathered on the device, in stream order."""
        R, B = self.rows, len(plan.slots)
        hv = self.hv
        self.copied.synchronize()              # the copy of the step before has left the pinned buffer
        hv[:4 * R] = 0
        hv[R:2 * R] = -1
        hv[3 * R:4 * R] = cache.padding_slot
        hv[0:B] = plan.flat
        hv[R:R + B] = plan.old
        hv[2 * R:2 * R + B] = plan.new_len
        hv[3 * R:3 * R + B] = plan.slots
        off = 4 * R
        for g, w in enumerate(self.widths):
            # the page tables change only when a sequence begins a page or the batch changes
            sig = cache.pages_signature(g, plan.slots)
            if sig != self.table_sig[g]:
                view = hv[off:off + R * w].reshape(R, w)
                view[:] = 0
                pages = cache.kv_groups[g].pages
                for r, s in enumerate(plan.slots):
                    l = pages[s]
                    if len(l) > w:
                        raise CacheError("page table width is too small")
                    view[r, :len(l)] = l
                self.table_sig[g] = sig
            off += R * w
        hv[off:self.pick_off] = -1
        for g in range(len(self.widths)):
            hv[off + g * R:off + g * R + B] = cache.decode_rows(g, plan.slots, plan.old)
        if ids is not None:
            hv[self.pick_off:self.pick_off + B] = pick
        if debug.ENABLED:
            tables, o = [], 4 * R
            for w in self.widths:
                tables.append(hv[o:o + R * w].reshape(R, w))
                o += R * w
            _checked(cache, "decode", 1 << 62, None if ids is not None else hv[0:B], list(hv[3 * R:4 * R]), hv[R:2 * R],
                     np.arange(R), hv[2 * R:3 * R], tables, [hv[off + g * R:off + (g + 1) * R] for g in range(len(self.widths))],
                     None)
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()
        if ids is not None:
            torch.index_select(ids, 0, self.pick[:B], out=self.tokens[:B])
        self.graph.replay()
        kernels.add_launches(self.kernels)
        return self.logits


class Engine:
    """A model with a cache: slots, steps, and nothing else."""

    def __init__(self, model: DecoderModel, max_tokens: int, max_slots: Optional[int] = None,
                 max_seq_len: Optional[int] = None, use_graphs: bool = True):
        self.model = model
        self.cache: Cache = model.new_cache(max_tokens, max_slots, max_seq_len)
        self.device = model.device
        self.vocab = model.layout.embedding.vocab
        parts = [p for blk in model.blocks for p in blk.parts().values() if p is not None] + [model.final_norm]
        self.use_graphs = bool(use_graphs and self.device.type == "cuda" and all(p.graph_safe for p in parts))
        self._graphs: dict[tuple, _DecodeGraph] = {}
        self._graphs_generation = model.generation
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs else None
        self.last_h2d_bytes = 0          # bytes the last step copied from the host
        self._pin: Optional[torch.Tensor] = None      # pinned staging buffer of the steps that are not captured
        self._pin_copied = None

    # slots ----------------------------------------------------------------
    def open(self, n: int = 1) -> list[int]:
        """Take n empty slots (all or none)."""
        if n > self.cache.slots.free_slots:
            raise CacheError(f"{n} sequences asked for, {self.cache.slots.free_slots} slots free")
        return [self.cache.alloc_slot() for _ in range(n)]

    def close(self, slots: Sequence[int]) -> None:
        for s in slots:
            self.cache.free_slot(s)
        # decode steps are queued without a look at the kernels' status words (that would cost a
        # synchronisation per step); the end of a batch is where a wait that ran out is reported
        self._check_waits("close", "the tokens decoded for these sequences are not valid")

    def _check_waits(self, where: str, consequence: str) -> None:
        """Raise if a bounded wait inside one of the tcgen05 kernels ran out since the last check.
        Reads and resets every status word (each read waits for the device)."""
        if self.device.type != "cuda" or self.model.dtype != torch.bfloat16:
            return
        codes = {"gemm_tc": kernels.gemm_tc_status(reset=True), "attn_tc": kernels.attention_tc_status(reset=True),
                 "gemm_stream": kernels.gemm_stream_status(reset=True)}
        bad = {k: v for k, v in codes.items() if v}
        if bad:
            raise StepError(f"{where}: a wait inside a tensor-core kernel ran out ({bad}), in this step or in a "
                            f"decode step since the last check; {consequence}")

    # the step -------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None, hidden: bool = False):
        """Run ``tokens[i]`` on ``slots[i]``; return logits [wanted, vocab] (float32, device).

        ``want[i]`` lists the places among ``tokens[i]`` whose logits are
        wanted (default: the last one of each), in the order given.  The
        result of a decode step is valid until the next step.

        ``hidden=True`` returns ``(logits, rows)``, ``rows`` being what the
        output matrix was given for the wanted places: the hidden state after
        the final norm, [wanted, hidden] in the step's element type
        (wlejon/brolm's ``hidden_out``, include/brolm/gemma2.h:121-125).
        """
        plan = self._plan(slots, tokens, want)
        if plan.mode == "decode" and self.use_graphs:
            graph = self._graph_for(plan)
            logits = graph.run(plan, self.cache)
            rows_h = graph.hidden
            self.last_h2d_bytes = graph.host.numel() * 4
            if plan.rows != list(range(len(plan.slots))):
                pick = torch.tensor(plan.rows, dtype=torch.long, device=self.device)
                logits, rows_h = logits[pick], rows_h[pick]
            else:
                logits, rows_h = logits[:len(plan.slots)], rows_h[:len(plan.slots)]
        else:
            ctx, tok_dev, rows = self._context(plan)
            logits = self.model.forward(ctx, tok_dev, rows)
            rows_h = self.model.last_hidden
            if plan.mode == "prefill":
                self._check_waits("step", "the results of this step are not valid")
        self.cache.commit(dict(zip(plan.slots, plan.new_len)))
        return (logits, rows_h) if hidden else logits

    def step_from(self, slots: Sequence[int], ids: torch.Tensor, pick: Sequence[int]) -> torch.Tensor:
        """A decode step whose tokens are still on the device: sequence ``slots[i]`` goes on with
        ``ids[pick[i]]``, ``ids`` being an int32 tensor that a sampler wrote.  Nothing waits for the
        values, so the step can be queued before the host has seen them; the logits are those of
        ``step`` with the same tokens."""
        if ids.dtype != torch.int32 or ids.dim() != 1 or ids.device != self.device:
            raise StepError("step_from: ids must be a one-dimensional int32 tensor on the engine's device")
        if len(pick) != len(slots) or any(not 0 <= int(p) < ids.numel() for p in pick):
            raise StepError("step_from: one place in ids per slot")
        plan = self._plan(slots, [[0]] * len(slots), None)
        if plan.mode != "decode":
            raise StepError("step_from: only sequences that already hold tokens can go on")
        if self.use_graphs:
            graph = self._graph_for(plan)
            logits = graph.run(plan, self.cache, ids, [int(p) for p in pick])[:len(plan.slots)]
            self.last_h2d_bytes = graph.host.numel() * 4
        else:
            ctx, _, rows = self._context(plan)
            tokens = ids.index_select(0, torch.tensor([int(p) for p in pick], dtype=torch.int32, device=self.device))
            logits = self.model.forward(ctx, tokens, rows)
        self.cache.commit(dict(zip(plan.slots, plan.new_len)))
        return logits

    def _graph_for(self, plan: _Plan) -> _DecodeGraph:
        if self._graphs_generation != self.model.generation:
            # the model's tensors were replaced (weights loaded again): the captured steps point at the old ones
            self._graphs.clear()
            self._graphs_generation = self.model.generation
        rows = _next_pow2(len(plan.slots))
        kv_cap = min(max(256, _next_pow2(max(plan.new_len))), _next_pow2(self.cache.max_positions))
        # sequences of very unequal lengths get a step of their own: its attention cuts every sequence
        # into more pieces than one round of blocks needs, so that the SMs even out what the lengths do not
        ragged = _ragged(plan.new_len)
        key = (rows, kv_cap, ragged)
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = _DecodeGraph(self, rows, kv_cap, ragged)
        return g

    def _plan(self, slots, tokens, want) -> _Plan:
        B = len(slots)
        if B == 0 or len(tokens) != B:
            raise StepError("step: needs as many token lists as slots, and at least one")
        if len(set(slots)) != B:
            raise StepError("step: a slot is named twice")
        cache = self.cache
        old = [cache.length(s) for s in slots]
        n_new = [len(t) for t in tokens]         # (lists, NumPy arrays and host tensors all have a length)
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
        try:
            flat = np.concatenate([np.asarray(seq, dtype=np.int64).reshape(-1) for seq in tokens])
        except (TypeError, ValueError, OverflowError):
            raise StepError("step: tokens must be sequences of integer ids") from None
        if flat.min() < 0 or flat.max() >= self.vocab:
            raise StepError(f"step: token id out of range [0, {self.vocab})")
        if want is None:
            want = [[n - 1] for n in n_new]
        if len(want) != B:
            raise StepError("step: 'want' needs one list per sequence")
        rows, start = [], 0
        for i, w in enumerate(want):
            for p in w:
                if not 0 <= p < n_new[i]:
                    raise StepError(f"step: wanted place {p} is outside the {n_new[i]} tokens given")
                rows.append(start + p)
            start += n_new[i]
        cache.reserve(dict(zip(slots, new_len)))
        return _Plan(mode, list(slots), n_new, old, new_len, flat, rows)

    def _context(self, plan: _Plan):
        cache, B = self.cache, len(plan.slots)
        T = int(sum(plan.n_new))
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(plan.n_new, out=cu[1:])
        positions = np.concatenate([np.arange(o, o + n) for o, n in zip(plan.old, plan.n_new)])
        tok_seq = np.repeat(np.arange(B), plan.n_new)
        tables = [cache.page_table(g, plan.slots).numpy() for g in range(len(cache.kv_groups))]
        # one host buffer, one copy
        parts = [plan.flat, positions, tok_seq, cu, np.asarray(plan.new_len), np.asarray(plan.slots),
                 np.asarray(plan.rows, dtype=np.int64)]
        parts += [t.reshape(-1) for t in tables]
        parts += [cache.write_rows(g, plan.slots, plan.old, plan.new_len) for g in range(len(tables))]
        if debug.ENABLED:
            _checked(cache, plan.mode, self.vocab, plan.flat, plan.slots, positions, tok_seq, np.asarray(plan.new_len),
                     tables, parts[7 + len(tables):], np.asarray(plan.rows, dtype=np.int64))
        sizes = [p.size for p in parts]
        offs = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])])
        n = int(offs[-1])
        if self.device.type == "cuda":
            # one pinned buffer for the engine's life (allocating pinned memory costs more than filling it);
            # the copy of the step before must have left it before it is written again
            if self._pin is None or self._pin.numel() < n:
                self._pin = torch.zeros(max(n, 4096), dtype=torch.int32, pin_memory=True)
                self._pin_copied = torch.cuda.Event()
            else:
                self._pin_copied.synchronize()
            host = self._pin[:n]
        else:
            host = torch.zeros(n, dtype=torch.int32)
        hv = host.numpy()
        hv[:] = 0
        for p, o in zip(parts, offs[:-1]):
            hv[o:o + p.size] = p
        dev = host.to(self.device, non_blocking=True)
        if self.device.type == "cuda":
            self._pin_copied.record()
        self.last_h2d_bytes = host.numel() * 4
        seg = [dev[int(o):int(o) + s] for o, s in zip(offs[:-1], sizes)]
        page_tables = [seg[7 + g].view(B, tables[g].shape[1]) for g in range(len(tables))]
        cache_rows = [seg[7 + len(tables) + g] for g in range(len(tables))]
        ctx = StepContext(mode=plan.mode, dtype=self.model.dtype, device=self.device, cache=cache, batch=B,
                          n_tokens=T, slots=plan.slots, positions=seg[1], tok_seq=seg[2], cu_q=seg[3],
                          kv_len=seg[4], slots_dev=seg[5], max_q_len=int(max(plan.n_new)), page_tables=page_tables,
                          cache_rows=cache_rows, host_lengths=plan.new_len,
                          ragged=plan.mode == "decode" and _ragged(plan.new_len))
        return ctx, seg[0], seg[6]
