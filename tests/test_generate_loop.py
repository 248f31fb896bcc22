"""The generation loop's decisions, with a scripted model in place of the GPU."""
import pytest
import torch

import brolm_b200 as bb
from brolm_b200.engine.generate import generate, plan_batches


class ScriptedEngine:
    """Predicts (last token + 1) % vocab; records what it was asked to do."""

    class _Cache:
        page_size = 64

        def __init__(self, max_tokens, max_slots):
            self.max_tokens, self.max_slots = max_tokens, max_slots

    def __init__(self, vocab=50, max_tokens=64 * 4, max_slots=4):
        self.vocab, self.cache = vocab, self._Cache(max_tokens, max_slots)
        self.free = list(range(max_slots))
        self.lengths = {}
        self.steps = []            # (mode, slots, lengths of the token lists)
        self.opened = []

    def open(self, n):
        assert n <= len(self.free)
        got = [self.free.pop(0) for _ in range(n)]
        for s in got:
            self.lengths[s] = 0
        self.opened.append(got)
        return got

    def close(self, slots):
        for s in slots:
            del self.lengths[s]
            self.free.append(s)

    def step(self, slots, tokens, want=None):
        fresh = [self.lengths[s] == 0 for s in slots]
        assert all(fresh) or (not any(fresh) and all(len(t) == 1 for t in tokens))
        self.steps.append(("prefill" if all(fresh) else "decode", list(slots), [len(t) for t in tokens]))
        out = torch.full((len(slots), self.vocab), -1.0)
        for r, (s, t) in enumerate(zip(slots, tokens)):
            self.lengths[s] += len(t)
            out[r, (t[-1] + 1) % self.vocab] = 1.0
        return out


def argmax_sampler(logits, streams, counter):
    return torch.argmax(logits, dim=-1)


def opts(n, **kw):
    return bb.GenerateOptions(max_new_tokens=n, sampling=bb.SamplingParams(temperature=0.0), **kw)


def test_counts_up_and_returns_only_new_tokens():
    e = ScriptedEngine()
    out = generate(e, [[3], [10, 11], [7, 8, 9]], eos_id=-1, opts=opts(4), sampler=argmax_sampler)
    assert out == [[4, 5, 6, 7], [12, 13, 14, 15], [10, 11, 12, 13]]
    assert e.steps[0] == ("prefill", [0, 1, 2], [1, 2, 3])
    assert [s[0] for s in e.steps[1:]] == ["decode"] * 3 and not e.lengths          # all slots given back


def test_stop_token_ends_one_sequence_and_is_not_returned():
    e = ScriptedEngine()
    out = generate(e, [[3], [20]], eos_id=6, opts=opts(5), sampler=argmax_sampler)
    assert out == [[4, 5], [21, 22, 23, 24, 25]]
    assert [s[1] for s in e.steps] == [[0, 1], [0, 1], [0, 1], [1], [1]]           # the shorter one left early
    out = generate(e, [[5]], eos_id=6, opts=opts(5), sampler=argmax_sampler)
    assert out == [[]]                                                               # eos first: nothing returned


def test_eos_can_be_switched_off_and_more_stop_ids_given():
    e = ScriptedEngine()
    assert generate(e, [[3]], eos_id=5, opts=opts(3, stop_on_eos=False), sampler=argmax_sampler) == [[4, 5, 6]]
    assert generate(e, [[3]], eos_id=-1, opts=opts(3), sampler=argmax_sampler) == [[4, 5, 6]]
    assert generate(e, [[3]], eos_id=40, opts=opts(9, stop_ids=(7,)), sampler=argmax_sampler) == [[4, 5, 6]]


def test_empty_prompt_and_zero_budget_give_nothing():
    e = ScriptedEngine()
    assert generate(e, [[], [1]], eos_id=-1, opts=opts(2), sampler=argmax_sampler) == [[], [2, 3]]
    assert e.steps[0][1] == [0]                                                      # the empty one took no slot
    assert generate(e, [[1], [2]], eos_id=-1, opts=opts(0), sampler=argmax_sampler) == [[], []]


def test_more_requests_than_slots_run_batch_after_batch():
    e = ScriptedEngine(max_slots=2)
    out = generate(e, [[i] for i in range(5)], eos_id=-1, opts=opts(2), sampler=argmax_sampler)
    assert out == [[i + 1, i + 2] for i in range(5)]
    assert e.opened == [[0, 1], [0, 1], [0]]                                         # slots used again
    assert [s[0] for s in e.steps] == ["prefill", "decode"] * 3


def test_batches_fit_the_cache():
    assert plan_batches([10, 10, 100, 10], 10, max_tokens=256, max_slots=8, page_size=64) == [[0, 1, 2], [3]]
    assert plan_batches([10, 0, 10], 10, max_tokens=1024, max_slots=8, page_size=64, batch_size=1) == [[0], [2]]
    with pytest.raises(ValueError):
        plan_batches([300], 10, max_tokens=256, max_slots=8, page_size=64)


def test_streams_follow_the_request_not_the_batch():
    e = ScriptedEngine(max_slots=2)
    seen = []

    def spy(logits, streams, counter):
        seen.append((streams.tolist(), counter))
        return torch.argmax(logits, dim=-1)

    generate(e, [[1], [2], [3]], eos_id=-1, opts=opts(2), sampler=spy)
    assert seen == [([0, 1], 0), ([0, 1], 1), ([2], 0), ([2], 1)]
