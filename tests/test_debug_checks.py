"""The checks of a step's description that ``BROLM_DEBUG=1`` switches on: right steps pass, and every
kind of wrong index is named before anything would be launched.  Host only."""
import numpy as np
import pytest

import brolm_b200 as bb
from brolm_b200.engine import debug
from brolm_b200.engine.model import DecoderModel
from brolm_b200.engine.step import StepError
from tests.helpers import TINY


@pytest.fixture()
def engine(monkeypatch):
    monkeypatch.setattr(debug, "ENABLED", True)
    cfg = bb.Gemma2Config(**TINY["B"][0])          # a window of 16: rings of one page
    model = DecoderModel(cfg, "float32", "cpu")
    return bb.Engine(model, max_tokens=64 * 6, max_slots=3, use_graphs=False), cfg


def _describe(eng, slots, tokens):
    """The host half of a step: plan, arrays, commit (nothing runs on a device)."""
    plan = eng._plan(slots, tokens, None)
    eng._context(plan)
    eng.cache.commit(dict(zip(plan.slots, plan.new_len)))
    return plan


def test_right_steps_pass(engine):
    eng, cfg = engine
    V = cfg.vocab_size
    a, b = eng.open(2)
    _describe(eng, [a, b], [list(range(1, 41)), [5, 6, 7]])          # 40 tokens: beyond the window's ring of 64? no; beyond the window
    for i in range(70):                                               # and across the ring's end and a page boundary
        _describe(eng, [a, b], [[(i * 7) % V], [(i * 3) % V]])
    eng.close([a, b])
    (c,) = eng.open(1)
    _describe(eng, [c], [list(range(2, 150))])                        # a prompt longer than the ring
    eng.close([c])


def _arrays(eng, slots, new_tokens):
    """What ``_context`` would hand to the check, as arrays that a test can spoil."""
    cache = eng.cache
    old = [cache.length(s) for s in slots]
    new = [o + len(t) for o, t in zip(old, new_tokens)]
    cache.reserve(dict(zip(slots, new)))
    positions = np.concatenate([np.arange(o, n) for o, n in zip(old, new)])
    tok_seq = np.repeat(np.arange(len(slots)), [len(t) for t in new_tokens])
    tables = [cache.page_table(g, slots).numpy().copy() for g in range(len(cache.kv_groups))]
    crows = [cache.write_rows(g, slots, old, new).copy() for g in range(len(cache.kv_groups))]
    tokens = np.concatenate([np.asarray(t) for t in new_tokens])
    return dict(cache=cache, mode="prefill" if all(o == 0 for o in old) else "decode", vocab=eng.vocab, tokens=tokens,
                slots=list(slots), positions=positions, tok_seq=tok_seq, kv_len=np.asarray(new), page_tables=tables,
                cache_rows=crows, wanted=np.asarray([len(tokens) - 1]))


@pytest.mark.parametrize("spoil,says", [
    (lambda k: k["tokens"].__setitem__(3, k["vocab"]), "token id"),
    (lambda k: k["positions"].__setitem__(2, 10 ** 6), "position"),
    (lambda k: k["kv_len"].__setitem__(0, k["kv_len"][0] + 1), "last position"),
    (lambda k: k["page_tables"][0].__setitem__((0, 0), 10 ** 5), "outside the pool"),
    (lambda k: k["page_tables"][0].__setitem__((0, 0), k["page_tables"][0][1, 0]), "differs from the pages"),
    (lambda k: k["cache_rows"][0].__setitem__(1, 10 ** 7), "outside the pool"),
    (lambda k: k["cache_rows"][0].__setitem__(1, k["cache_rows"][0][0]), "one place"),
    (lambda k: k["cache_rows"][1].__setitem__(slice(4, 6), k["cache_rows"][1][4:6][::-1].copy()), "lives at"),
    (lambda k: k["cache_rows"][0].__setitem__(0, -1), "not kept"),
    (lambda k: k["wanted"].__setitem__(0, 10 ** 4), "wanted row"),
    (lambda k: k["slots"].__setitem__(1, 2), "no sequence holds"),
    (lambda k: k["slots"].__setitem__(1, k["slots"][0]), "two rows"),
])
def test_every_kind_of_wrong_index_is_named(engine, spoil, says):
    eng, cfg = engine
    a, b = eng.open(2)
    kw = _arrays(eng, [a, b], [list(range(1, 31)), list(range(3, 12))])
    debug.check_step(**kw)                                            # as made: fine
    spoil(kw)
    with pytest.raises(debug.StepCheckError, match=says):
        debug.check_step(**kw)


def test_a_spoilt_cache_stops_the_step(engine):
    """The engine's own path: a page that two sequences hold (here put there by hand) raises StepError
    from ``step`` itself, before any copy or launch."""
    eng, cfg = engine
    a, b = eng.open(2)
    _describe(eng, [a, b], [list(range(1, 9)), list(range(1, 9))])
    g = eng.cache.kv_groups[0]
    g.pages[b][0] = g.pages[a][0]
    with pytest.raises(StepError, match="debug: group 0"):
        plan = eng._plan([a, b], [[1], [2]], None)
        eng._context(plan)
