"""Schedules that long runs and real sizes reach, each against the plain implementation:

* a sequence whose captured decode step changes from one length bucket to the next while it is
  decoded, alone, beside shorter ones, and in the very step in which the batch shrinks to another
  padded size;
* two layers at the Gemma 2 2B layer sizes with the real window of 4,096 keys: a prompt longer
  than the window, decode steps over the full ring, and a shorter prompt decoded across the
  ring's end;
* sampled generation through the entry point against the plain forward pass and the plain sampler;
* the rows behind the logits (the hidden state after the final norm) from prompt and decode steps;
* two engines of one model, made one after the other with a growing number of positions, both
  decoding from captured steps;
* random weights made on the device and on the host: the same bits.
"""
import pytest
import torch

import brolm_b200 as bb
from brolm_b200.sampling import uniform24
from tests.helpers import TINY, make_folder, oracle_inputs, random_prompts
from tests.plain import gemma2_plain as plain
from tests.plain import sampling_plain
from tests.test_engine_gpu import STORE, TOL, check, run_batch_teacher_forced

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CASES = [(name, dtype) for name in ("A", "B") for dtype in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    out = {}
    for name, dtype in CASES:
        folder = make_folder(tmp, name, STORE[dtype])
        config, weights = oracle_inputs(folder)
        out[(name, dtype)] = (folder, config, weights, bb.load_model(folder, dtype=dtype, device=DEV))
    return out


@pytest.mark.parametrize("name,dtype", CASES)
def test_decoding_across_the_length_buckets_of_the_captured_step(setups, name, dtype):
    """Captured decode steps are kept per (padded batch, bound on the lengths: 256, 512, 1024, ...).
    A sequence that grows past a bound goes on in another captured step, with page tables made anew
    and another number of splits of its keys."""
    _, config, weights, model = setups[(name, dtype)]
    V = config["vocab_size"]
    eng = bb.Engine(model, max_tokens=4096, max_slots=4)
    assert eng.use_graphs
    for total, start in ((270, 250), (520, 505)):
        p = random_prompts(V, [total], seed=total)[0]
        ref = plain.forward(config, weights, p)
        (s,) = eng.open(1)
        check(eng.step([s], [p[:start]])[0], ref[start - 1], dtype, "prompt")
        for i in range(start, total):
            check(eng.step([s], [[p[i]]])[0], ref[i], dtype, f"token {i} of {total}")
        eng.close([s])
    caps = {key[1] for key in eng._graphs}
    assert {256, 512, 1024} <= caps, caps
    # members on both sides of 256; the longest crosses it while the others are still far below
    run_batch_teacher_forced(eng, config, weights, random_prompts(V, [262, 40, 258, 300], 5), [250, 30, 255, 290], dtype)
    # the batch shrinks from three sequences (four rows) to two in the very step in which the longest
    # reaches 257 tokens: another padded size and another bucket at once
    before = set(eng._graphs)
    run_batch_teacher_forced(eng, config, weights, random_prompts(V, [270, 7, 40], 6), [250, 1, 30], dtype)
    assert {(2, 512), (4, 256)} <= {key[:2] for key in eng._graphs}, (before, set(eng._graphs))
    # the batches of unequal lengths ran in captured steps of their own (more pieces per sequence in the attention)
    assert any(key[2] for key in eng._graphs) and any(not key[2] for key in eng._graphs)
    assert eng.cache.live_slots == 0


def test_real_window_at_the_2b_layer_sizes(tmp_path):
    """Two layers (one sliding, one global) with the sizes of Gemma 2 2B and sliding_window = 4096, bfloat16.
    The ring of the sliding layer then has 64 pages; a window that straddles a page boundary reads 65
    tiles from 64 pages, the first and the last from the same page."""
    cfg = bb.Gemma2Config(vocab_size=1000, num_hidden_layers=2)           # the defaults are the 2B sizes
    assert cfg.sliding_window == 4096 and cfg.hidden_size == 2304 and cfg.head_dim == 256
    folder = str(tmp_path / "two_layers")
    bb.write_random_model(cfg, folder, seed=2, dtype=torch.bfloat16, device=DEV)
    config, weights = oracle_inputs(folder)
    model = bb.load_model(folder, dtype="bfloat16", device=DEV)
    p = random_prompts(1000, [4208], seed=3)[0]
    ref = plain.forward(config, weights, p)
    eng = bb.Engine(model, max_tokens=4224 + 4224, max_slots=2)
    # a prompt longer than the window, then decode steps over the full ring
    (s,) = eng.open(1)
    got = eng.step([s], [p[:4200]], want=[list(range(4184, 4200))])
    check(got, ref[4184:4200], "bfloat16", "last rows of a prompt of 4,200 tokens")
    for i in range(4200, 4208):
        check(eng.step([s], [[p[i]]])[0], ref[i], "bfloat16", f"token {i} after a prompt beyond the window")
    # a prompt shorter than the window in a second slot, decoded across position 4096 and a page beyond it
    (t,) = eng.open(1)
    check(eng.step([t], [p[:3000]])[0], ref[2999], "bfloat16", "prompt of 3,000 tokens")
    worst = 0.0
    for i in range(3000, 4170):
        got = eng.step([t], [[p[i]]])
        if i % 16 == 0 or 4030 <= i:
            worst = max(worst, check(got[0], ref[i], "bfloat16", f"token {i}, decoded across the ring's end"))
    eng.close([s, t])
    assert worst > 0.0


@pytest.mark.parametrize("params", [dict(temperature=0.8, seed=7), dict(temperature=0.8, top_k=40, top_p=0.9, seed=7)])
def test_sampled_generation_is_plain_forward_plus_plain_sampler(setups, params):
    """Tiny B's own workload: four prompts of 1, 9, 23 and 40 tokens (beyond the window of 16), twelve
    tokens each at temperature 0.8 with seed 7, float32.  Every drawn token is what the plain sampler
    draws from the plain logits of the tokens so far with the same uniform number
    (wlejon/brolm src/detail/generate.cpp:68-142; its own test forces the teacher's tokens in the
    same way, tests/test_qwen_generate.cpp:282-323)."""
    _, config, weights, model = setups[("B", "float32")]
    sp = bb.SamplingParams(**params)
    eng = bb.Engine(model, max_tokens=64 * 4, max_slots=4)
    prompts = random_prompts(config["vocab_size"], [1, 9, 23, 40], seed=71)
    opts = bb.GenerateOptions(max_new_tokens=12, sampling=sp, stop_on_eos=False)
    outs = bb.generate(eng, prompts, eos_id=-1, opts=opts)
    for request, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o) == 12
        ids = list(p)
        for step, tok in enumerate(o):
            row = plain.forward(config, weights, ids)[-1]
            want = sampling_plain.sample(row, sp.temperature, sp.top_k, sp.top_p, uniform24(sp.seed, request, step))
            assert tok == want, (request, step)
            ids.append(tok)
    assert len({tuple(o) for o in outs}) == 4


@pytest.mark.parametrize("name,dtype", CASES)
def test_hidden_rows_behind_the_logits(setups, name, dtype):
    _, config, weights, model = setups[(name, dtype)]
    eng = bb.Engine(model, max_tokens=512, max_slots=3)
    prompts = random_prompts(config["vocab_size"], [40, 7, 21], seed=81)
    refs = [plain.hidden(config, weights, p) for p in prompts]
    pre = [30, 1, 20]
    slots = eng.open(3)
    want = [[0, k - 1] for k in pre]
    logits, rows = eng.step(slots, [p[:k] for p, k in zip(prompts, pre)], want=want, hidden=True)
    assert rows.shape == (6, config["hidden_size"]) and logits.shape[0] == 6
    for i, (r, k) in enumerate(zip(refs, pre)):
        check(rows[2 * i], r[0], dtype, "first row of a prompt")
        check(rows[2 * i + 1], r[k - 1], dtype, "last row of a prompt")
    for step in range(3):
        live = [i for i in range(3) if pre[i] + step < len(prompts[i])]
        logits, rows = eng.step([slots[i] for i in live], [[prompts[i][pre[i] + step]] for i in live], hidden=True)
        assert rows.shape == (len(live), config["hidden_size"])
        for row, i in enumerate(live):
            check(rows[row], refs[i][pre[i] + step], dtype, "row of a decode step")
    eng.close(slots)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_engines_of_one_model_with_growing_positions(setups, dtype):
    """The rotary table belongs to the model's position part and grows when a later engine asks for more
    positions; the captured steps of the earlier engine keep reading the table they were captured with."""
    _, config, weights, model = setups[("A", dtype)]
    V = config["vocab_size"]
    p = random_prompts(V, [60], seed=91)[0]
    q = random_prompts(V, [900], seed=92)[0]
    ref_p, ref_q = plain.forward(config, weights, p), plain.forward(config, weights, q)
    small = bb.Engine(model, max_tokens=128, max_slots=1)
    (a,) = small.open(1)
    small.step([a], [p[:20]])
    for i in range(20, 30):
        check(small.step([a], [[p[i]]])[0], ref_p[i], dtype, "first engine, before the second exists")
    large = bb.Engine(model, max_tokens=1024, max_slots=1)            # more positions: the table is made anew
    # whatever the second engine's set-up freed is taken again and overwritten: blocks of the old table's size
    # (the allocator keeps small and large blocks apart) and a few large ones
    old_bytes = 128 * (config["head_dim"] // 2) * 2 * 4
    filler = [torch.empty(old_bytes // 4, device=DEV) for _ in range(256)] + [torch.empty(1 << 20, device=DEV) for _ in range(8)]
    for f in filler:
        f.fill_(float("nan"))
    (b,) = large.open(1)
    large.step([b], [q[:880]])
    for i in range(30, 60):
        check(small.step([a], [[p[i]]])[0], ref_p[i], dtype, "first engine, after the table grew")
        if i < 50:
            j = 880 + i - 30
            check(large.step([b], [[q[j]]])[0], ref_q[j], dtype, "second engine")
    small.close([a])
    large.close([b])


@pytest.mark.parametrize("name,dtype", [("A", "bfloat16"), ("B", "bfloat16"), ("B", "float32")])
def test_many_random_batches_one_after_another(setups, name, dtype):
    """Twelve batches of one to five requests with random prompt lengths, random prefill cuts and random
    decode lengths through one engine, every logit against the plain implementation: equal and very
    unequal lengths in turn (both kinds of captured step), batches that shrink step by step, slots and
    pages used again and again, lengths on both sides of the captured steps' bounds and of the ring."""
    import random
    _, config, weights, model = setups[(name, dtype)]
    V = config["vocab_size"]
    rng = random.Random(1234 + len(name) + len(dtype))
    eng = bb.Engine(model, max_tokens=64 * 24, max_slots=5)
    for batch in range(12):
        n = rng.randint(1, 5)
        lengths = [rng.choice((rng.randint(2, 40), rng.randint(40, 140), rng.randint(240, 300))) for _ in range(n)]
        prefill = [rng.randint(1, max(1, L - rng.randint(1, 24))) for L in lengths]
        run_batch_teacher_forced(eng, config, weights, random_prompts(V, lengths, 500 + batch), prefill, dtype)
        assert eng.cache.live_slots == 0 and all(g.pool.held_pages == 0 for g in eng.cache.kv_groups)
    if eng.use_graphs:
        assert any(key[2] for key in eng._graphs) and any(not key[2] for key in eng._graphs)


@pytest.mark.parametrize("graphs", [True, False])
def test_steps_pass_the_debug_checks(setups, monkeypatch, graphs):
    """With the checks of BROLM_DEBUG=1 on, prompts longer than the window's ring, unequal batches one after
    the other (slots and pages used again) and decoding across the ring's end run as ever: the checks
    find nothing in right steps, through the captured decode step and without it."""
    from brolm_b200.engine import debug
    monkeypatch.setattr(debug, "ENABLED", True)
    _, config, weights, model = setups[("B", "bfloat16")]
    V = config["vocab_size"]
    eng = bb.Engine(model, max_tokens=64 * 12, max_slots=3, use_graphs=graphs)
    assert eng.use_graphs == graphs
    run_batch_teacher_forced(eng, config, weights, random_prompts(V, [90, 7, 40], 31), [70, 1, 30], "bfloat16")
    run_batch_teacher_forced(eng, config, weights, random_prompts(V, [33, 140], 32), [20, 130], "bfloat16")
    assert eng.cache.live_slots == 0


def test_random_weights_are_the_same_bits_on_the_host_and_on_the_device():
    from brolm_b200.weights.random_init import random_tensor
    for dtype in (torch.float32, torch.bfloat16):
        for name, shape, std in (("model.embed_tokens.weight", (1000, 2304), 0.02), ("model.norm.weight", (2304,), 0.1),
                                 ("x", (3, 5, 7), 1.0)):
            host = random_tensor(11, name, shape, std, dtype, "cpu")
            dev = random_tensor(11, name, shape, std, dtype, DEV)
            assert torch.equal(host, dev.cpu())
    cfg = bb.Gemma2Config(**TINY["A"][0])
    a = bb.Model(cfg, dtype="bfloat16", device=DEV).init_random(seed=4, on_device=True)
    b = bb.Model(cfg, dtype="bfloat16", device=DEV).init_random(seed=4, on_device=False)
    assert torch.equal(a.embedding, b.embedding)
    assert torch.equal(a.blocks[1].feedforward.w_down, b.blocks[1].feedforward.w_down)
    assert torch.equal(a.blocks[0].pre_mixer_norm.weight, b.blocks[0].pre_mixer_norm.weight)
