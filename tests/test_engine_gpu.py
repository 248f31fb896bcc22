"""The engine against the plain implementation, in float32 and in bfloat16:
whole requests, the last 32 tokens one by one, batches of unequal lengths
whose shorter requests end earlier (batch after batch, so that slots and pages
are used again), long decoding past the window's ring, the first tokens of a
sequence, and greedy generation through the entry point."""
import os

import pytest
import torch

import brolm_b200 as bb
from tests.helpers import TINY, make_folder, oracle_inputs, random_prompts
from tests.plain import gemma2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# Largest error of a logit against the float64 oracle, relative to the largest
# logit of the compared rows.  Measured on whole requests of up to 300 tokens:
# float32 5e-7 and 7e-7 for the two tiny models, bfloat16 6e-3 and 8e-3 (8-bit
# mantissas in weights, activations and cache).  wlejon/brolm's own bars are
# 1e-4 absolute for its float path and 5e-2 for 16 bits
# (tests/test_gemma2.cpp:247-248).
TOL = {"float32": 1e-5, "bfloat16": 2e-2}
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}

CASES = [(name, dtype) for name in ("A", "B", "C") for dtype in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    out = {}
    for name, dtype in CASES:
        folder = make_folder(tmp, name, STORE[dtype])
        config, weights = oracle_inputs(folder)
        model = bb.load_model(folder, dtype=dtype, device=DEV)
        out[(name, dtype)] = (folder, config, weights, model)
    return out


def check(got, ref, dtype, what):
    ref = ref.double()
    err = float((got.double().cpu() - ref).abs().max()) / max(float(ref.abs().max()), 1e-3)
    assert err <= TOL[dtype], f"{what}: relative error {err:.3e} exceeds {TOL[dtype]:.0e}"
    return err


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_requests(setups, name, dtype):
    _, config, weights, model = setups[(name, dtype)]
    eng = bb.Engine(model, max_tokens=512)
    for p in random_prompts(config["vocab_size"], [1, 5, 64, 65, 150], seed=11):
        ref = plain.forward(config, weights, p)
        (s,) = eng.open(1)
        got = eng.step([s], [p], want=[list(range(len(p)))])
        check(got, ref, dtype, f"whole request of {len(p)}")
        assert float(got.abs().max()) <= config["final_logit_softcapping"]
        eng.close([s])


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(setups, name, dtype):
    _, config, weights, model = setups[(name, dtype)]
    eng = bb.Engine(model, max_tokens=512)
    for p in random_prompts(config["vocab_size"], [40, 100, 170], seed=12):
        ref = plain.forward(config, weights, p)
        (s,) = eng.open(1)
        n = len(p) - 32
        got = eng.step([s], [p[:n]], want=[list(range(n))])
        check(got, ref[:n], dtype, "prompt part")
        for i in range(n, len(p)):
            got = eng.step([s], [[p[i]]])
            check(got[0], ref[i], dtype, f"token {i} of {len(p)} decoded alone")
        eng.close([s])


def run_batch_teacher_forced(eng, config, weights, prompts, prefill, dtype):
    """Prefill ``prefill[i]`` tokens of each prompt together, then feed each
    request's own next token; a request that runs out leaves the batch."""
    refs = [plain.forward(config, weights, p) for p in prompts]
    slots = eng.open(len(prompts))
    got = eng.step(slots, [p[:k] for p, k in zip(prompts, prefill)], want=[list(range(k)) for k in prefill])
    off = 0
    for r, k in zip(refs, prefill):
        check(got[off:off + k], r[:k], dtype, "batched prompt")
        off += k
    done = list(prefill)
    live = [i for i in range(len(prompts)) if done[i] < len(prompts[i])]
    for i in range(len(prompts)):
        if i not in live:
            eng.close([slots[i]])
    while live:
        got = eng.step([slots[i] for i in live], [[prompts[i][done[i]]] for i in live])
        for row, i in enumerate(live):
            check(got[row], refs[i][done[i]], dtype, f"request {i} token {done[i]} in a batch of {len(live)}")
            done[i] += 1
        for i in live:
            if done[i] >= len(prompts[i]):
                eng.close([slots[i]])
        live = [i for i in live if done[i] < len(prompts[i])]


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_one_after_another(setups, name, dtype):
    _, config, weights, model = setups[(name, dtype)]
    # room for one batch at a time only: the second and third batch must reuse slots and pages
    eng = bb.Engine(model, max_tokens=64 * 8, max_slots=4)
    V = config["vocab_size"]
    run_batch_teacher_forced(eng, config, weights, random_prompts(V, [9, 100, 40, 150], 21), [5, 90, 1, 140], dtype)
    assert eng.cache.live_slots == 0
    run_batch_teacher_forced(eng, config, weights, random_prompts(V, [130, 3, 70, 66], 22), [120, 3, 64, 30], dtype)
    run_batch_teacher_forced(eng, config, weights, random_prompts(V, [33, 34], 23), [1, 2], dtype)
    assert eng.cache.live_slots == 0
    assert all(g.pool.held_pages == 0 for g in eng.cache.kv_groups)


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding_from_a_short_prompt(setups, name, dtype):
    _, config, weights, model = setups[(name, dtype)]
    eng = bb.Engine(model, max_tokens=512)
    p = random_prompts(config["vocab_size"], [210], seed=31)[0]
    ref = plain.forward(config, weights, p)
    (s,) = eng.open(1)
    got = eng.step([s], [p[:1]])
    check(got[0], ref[0], dtype, "first token")
    for i in range(1, len(p)):
        got = eng.step([s], [[p[i]]])
        check(got[0], ref[i], dtype, f"token {i}")
    eng.close([s])


@pytest.mark.parametrize("name,dtype", CASES)
def test_padding_changes_nothing(setups, name, dtype):
    """The same request gives the same logits alone and beside others of any length."""
    _, config, weights, model = setups[(name, dtype)]
    eng = bb.Engine(model, max_tokens=1024)
    ps = random_prompts(config["vocab_size"], [70, 3, 129], seed=41)
    (s,) = eng.open(1)
    alone = eng.step([s], [ps[0]], want=[list(range(70))]).clone()
    eng.close([s])
    slots = eng.open(3)
    together = eng.step(slots, ps, want=[list(range(70)), [], [128]])
    eng.close(slots)
    if dtype == "float32":
        assert torch.equal(alone, together[:70])
    else:
        assert float((alone - together[:70]).abs().max()) <= TOL[dtype] * float(alone.abs().max())


@pytest.mark.parametrize("name,dtype", CASES)
def test_greedy_generation_through_the_entry_point(setups, name, dtype):
    _, config, weights, model = setups[(name, dtype)]
    eng = bb.Engine(model, max_tokens=64 * 6, max_slots=3)
    prompts = random_prompts(config["vocab_size"], [5, 11, 17, 1, 70], seed=51)
    opts = bb.GenerateOptions(max_new_tokens=8, sampling=bb.SamplingParams(temperature=0.0), stop_on_eos=False)
    outs = bb.generate(eng, prompts, eos_id=-1, opts=opts)
    assert eng.cache.live_slots == 0
    for p, o in zip(prompts, outs):
        assert len(o) == 8
        if dtype == "float32":
            assert o == plain.greedy(config, weights, p, 8)
        else:
            # bfloat16 may pick another of two near-equal logits: the pick must be the oracle's
            # maximum within the tolerance, given the tokens generated so far
            ids = list(p)
            for tok in o:
                row = plain.forward(config, weights, ids)[-1]
                assert float(row.max() - row[tok]) <= 2 * TOL[dtype] * float(row.abs().max())
                ids.append(tok)


def test_step_refuses_a_mixed_batch(setups):
    _, config, weights, model = setups[("A", "float32")]
    eng = bb.Engine(model, max_tokens=256)
    a, b = eng.open(2)
    eng.step([a], [[1, 2, 3]])
    with pytest.raises(bb.StepError):
        eng.step([a, b], [[4], [5, 6]])
    with pytest.raises(bb.StepError):
        eng.step([a], [[4, 5]])
    with pytest.raises(bb.StepError):
        eng.step([b], [[config["vocab_size"]]])
    eng.close([a, b])


ODD = dict(vocab_size=257, hidden_size=100, intermediate_size=90, num_hidden_layers=2, num_attention_heads=5,
           num_key_value_heads=5, head_dim=48, rope_theta=5000.0, sliding_window=70, attn_logit_softcapping=0.0,
           final_logit_softcapping=0.0, query_pre_attn_scalar=48, rms_norm_eps=1e-6, max_position_embeddings=256)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_fit_no_fast_path(tmp_path, dtype):
    """A width that is no multiple of 8, an odd vocabulary, five heads of 48, no soft-caps at all, and a
    window that is no multiple of the page: every kernel has to take its general path or hand over."""
    folder = str(tmp_path / "odd")
    bb.write_random_model(bb.Gemma2Config(**ODD), folder, seed=5, weight_std=0.05, dtype=STORE[dtype])
    config, weights = oracle_inputs(folder)
    model = bb.load_model(folder, dtype=dtype, device=DEV)
    eng = bb.Engine(model, max_tokens=1024, max_slots=3)
    prompts = random_prompts(257, [150, 20, 71], seed=6)
    refs = [plain.forward(config, weights, p) for p in prompts]
    pre = [140, 1, 70]
    slots = eng.open(3)
    got = eng.step(slots, [p[:k] for p, k in zip(prompts, pre)], want=[list(range(k)) for k in pre])
    off = 0
    for r, k in zip(refs, pre):
        check(got[off:off + k], r[:k], dtype, "prompt")
        off += k
    for step in range(10):
        live = [i for i in range(3) if pre[i] + step < len(prompts[i])]
        got = eng.step([slots[i] for i in live], [[prompts[i][pre[i] + step]] for i in live])
        for row, i in enumerate(live):
            check(got[row], refs[i][pre[i] + step], dtype, f"decode {step} of request {i}")
    eng.close(slots)


def test_tensors_stored_in_32_bits_stay_so_and_still_compute(tmp_path):
    """bfloat16 run of a checkpoint in which some gains and one matrix are stored as float32."""
    from safetensors.torch import load_file, save_file
    folder = make_folder(tmp_path, "B", torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    for name in ("model.layers.0.post_attention_layernorm.weight", "model.norm.weight",
                 "model.layers.1.mlp.down_proj.weight", "model.layers.2.self_attn.k_proj.weight"):
        tensors[name] = tensors[name].float()
    save_file(tensors, path)
    config, weights = oracle_inputs(folder)
    model = bb.load_model(folder, dtype="bfloat16", device=DEV)
    assert model.final_norm.weight.dtype == torch.float32 and model.blocks[1].feedforward.w_down.dtype == torch.float32
    assert model.blocks[2].mixer.w_qkv.dtype == torch.float32 and model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    eng = bb.Engine(model, max_tokens=512)
    p = random_prompts(config["vocab_size"], [90], seed=8)[0]
    ref = plain.forward(config, weights, p)
    (s,) = eng.open(1)
    check(eng.step([s], [p[:80]], want=[list(range(80))]), ref[:80], "bfloat16", "prompt")
    for i in range(80, 90):
        check(eng.step([s], [[p[i]]])[0], ref[i], "bfloat16", f"token {i}")
    eng.close([s])


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_generation_one_step_ahead_equals_step_by_step(setups, graphs, temperature):
    """On a GPU the loop queues the next step from the ids on the device before the host has read them.
    With stop tokens that do occur, a budget that cuts requests off and more requests than slots, it
    returns what the step-by-step loop returns (float32: the same ids)."""
    _, config, weights, model = setups[("B", "float32")]
    V = config["vocab_size"]
    prompts = random_prompts(V, [5, 30, 17, 1, 70, 9, 2], seed=61)
    params = bb.SamplingParams(temperature=temperature, top_k=50 if temperature else 0, seed=7)

    def run(step_by_step, stop_ids, max_new):
        eng = bb.Engine(model, max_tokens=64 * 8, max_slots=3, use_graphs=graphs)
        opts = bb.GenerateOptions(max_new_tokens=max_new, sampling=params, stop_on_eos=True, stop_ids=stop_ids)
        sampler = bb.Sampler(params)
        if step_by_step:
            inner = sampler
            sampler = lambda logits, streams, counter: inner(logits, streams, counter)   # not a Sampler: no run-ahead
        out = bb.generate(eng, prompts, eos_id=-1, opts=opts, sampler=sampler)
        assert eng.cache.live_slots == 0
        return out

    free = run(True, [], 12)
    # stop ids taken from what is generated: some requests end early, at different steps
    stop_ids = sorted({o[3] for o in free[:3]} | {free[4][0]})
    for max_new in (1, 2, 12):
        a, b = run(True, stop_ids, max_new), run(False, stop_ids, max_new)
        assert a == b
        assert any(len(o) < max_new for o in a) or max_new == 1
        for o in a:
            assert not set(o) & set(stop_ids) and len(o) <= max_new


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("batch", [12, 20, 33, 64, 100])
def test_decode_in_wider_batches(setups, name, dtype, batch, monkeypatch):
    """Twelve sequences (two token tiles of the few-token products), then twenty to a hundred (the tcgen05
    weight stream with 32, 64 and 128 token columns; q/k/v as slices of K that the rotation adds): unequal
    prompts together, then token by token, against the plain implementation.  (By default more than 32
    tokens go to the library product; here the own kernel takes them all.)"""
    from brolm_b200 import kernels
    monkeypatch.setattr(kernels, "STREAM_ROWS", 128)
    _, config, weights, model = setups[(name, dtype)]
    V = config["vocab_size"]
    g = torch.Generator().manual_seed(batch)
    lengths = [int(x) for x in torch.randint(3, 40, (batch,), generator=g)]
    prompts = random_prompts(V, lengths, seed=70 + batch)
    eng = bb.Engine(model, max_tokens=64 * batch, max_slots=batch)
    run_batch_teacher_forced(eng, config, weights, prompts, [max(1, n - 4) for n in lengths], dtype)
    assert eng.cache.live_slots == 0
