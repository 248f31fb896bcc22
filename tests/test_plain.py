"""The plain implementation checked against itself and against the reference's own conventions."""
import math

import torch

from tests.plain import gemma2_plain as plain
from tests.plain import sampling_plain


def test_rms_norm_has_unit_rms_before_the_gain():
    x = torch.randn(5, 48, dtype=torch.float64) * 7
    y = plain.rms_norm(x, torch.zeros(48), 1e-12)
    assert torch.allclose((y * y).mean(-1), torch.ones(5, dtype=torch.float64), atol=1e-9)
    w = torch.randn(48) * 0.1
    assert torch.allclose(plain.rms_norm(x, w, 1e-12), y * (1 + w.double()))


def test_rope_is_a_rotation_and_depends_on_the_distance_only():
    hd, theta = 32, 1000.0
    q, k = torch.randn(1, hd, dtype=torch.float64), torch.randn(1, hd, dtype=torch.float64)
    for p, j in [(5, 2), (105, 102), (40, 37)]:
        qr = plain.rope(q, torch.tensor([p]), hd, theta)
        kr = plain.rope(k, torch.tensor([j]), hd, theta)
        assert abs(float(qr.norm()) - float(q.norm())) < 1e-9
        if (p, j) == (5, 2):
            first = float((qr * kr).sum())
        assert abs(float((qr * kr).sum()) - first) < 1e-9
    assert torch.equal(plain.rope(q, torch.tensor([0]), hd, theta), q)


def test_pairing_equals_the_references_permuted_adjacent_pairs():
    """brolm permutes the rows of Wq/Wk (dst rows 2i, 2i+1 <- src rows i, i + hd/2,
    include/brolm/detail/weights.h:106-127) and rotates adjacent pairs; scores are the same."""
    hd, heads, theta, T = 16, 3, 10000.0, 6
    g = torch.Generator().manual_seed(0)
    q = torch.randn(T, heads * hd, generator=g, dtype=torch.float64)
    k = torch.randn(T, heads * hd, generator=g, dtype=torch.float64)
    pos = torch.arange(T)

    def permute(x):                       # what the permuted projection would output
        x = x.reshape(T, heads, hd)
        out = torch.empty_like(x)
        out[..., 0::2] = x[..., :hd // 2]
        out[..., 1::2] = x[..., hd // 2:]
        return out.reshape(T, heads * hd)

    def rope_adjacent(x):                 # rotation of the pairs (2i, 2i+1) by pos * theta^(-2i/hd)
        x = x.reshape(T, heads, hd)
        i = torch.arange(hd // 2, dtype=torch.float64)
        ang = pos.double()[:, None] * theta ** (-2.0 * i / hd)
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = a * s + b * c
        return out.reshape(T, heads * hd)

    ours_q, ours_k = plain.rope(q, pos, hd, theta), plain.rope(k, pos, hd, theta)
    ref_q, ref_k = rope_adjacent(permute(q)), rope_adjacent(permute(k))
    for h in range(heads):
        sl = slice(h * hd, (h + 1) * hd)
        assert torch.allclose(ours_q[:, sl] @ ours_k[:, sl].t(), ref_q[:, sl] @ ref_k[:, sl].t(), atol=1e-12)


def test_attention_mask_and_groups():
    T, n_q, n_kv, hd = 9, 4, 2, 8
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(T, n * hd, generator=g, dtype=torch.float64) for n in (n_q, n_kv, n_kv))
    full = plain.attention(q, k, v, n_q, n_kv, hd, 0.3, 0.0, 0)
    assert torch.allclose(plain.attention(q, k, v, n_q, n_kv, hd, 0.3, 0.0, T), full)       # window >= T: no effect
    one = plain.attention(q, k, v, n_q, n_kv, hd, 0.3, 0.0, 1)                              # window 1: own value only
    assert torch.allclose(one.reshape(T, n_q, hd)[:, 3], v.reshape(T, n_kv, hd)[:, 1])     # head 3 reads kv head 1
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0.0, 9.0                                                               # the future does not matter
    assert torch.allclose(plain.attention(q, k2, v2, n_q, n_kv, hd, 0.3, 0.0, 0)[:5], full[:5])
    w3 = plain.attention(q, k, v, n_q, n_kv, hd, 0.3, 0.0, 3)
    k3 = k.clone()
    k3[2] += 100.0                                                                          # key 2 is outside the window of query 5
    assert torch.allclose(plain.attention(q, k3, v, n_q, n_kv, hd, 0.3, 0.0, 3)[5], w3[5])
    assert not torch.allclose(plain.attention(q, k3, v, n_q, n_kv, hd, 0.3, 0.0, 3)[4], w3[4])


def test_one_query_alone_is_the_last_row():
    T, n_q, n_kv, hd = 23, 6, 2, 8
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(T, n * hd, generator=g, dtype=torch.float64) for n in (n_q, n_kv, n_kv))
    for window, cap in ((0, 0.0), (5, 3.0), (23, 0.0), (40, 1.5), (1, 0.0)):
        whole = plain.attention(q, k, v, n_q, n_kv, hd, 0.4, cap, window)[-1]
        assert torch.allclose(plain.attention_last_query(q[-1], k, v, n_q, n_kv, hd, 0.4, cap, window), whole,
                              atol=1e-12)


def test_soft_cap_and_gelu():
    x = torch.linspace(-200, 200, 101, dtype=torch.float64)
    assert float(plain.soft_cap(x, 30.0).abs().max()) <= 30.0 and torch.equal(plain.soft_cap(x, 0.0), x)
    assert abs(float(plain.soft_cap(torch.tensor(1e-3, dtype=torch.float64), 50.0)) - 1e-3) < 1e-9
    z = torch.tensor([-3.0, 0.0, 0.5, 4.0], dtype=torch.float64)
    exact = 0.5 * z * (1 + torch.erf(z / math.sqrt(2)))
    assert float((plain.gelu_tanh(z) - exact).abs().max()) < 3e-3 and float(plain.gelu_tanh(z)[1]) == 0.0


def test_forward_is_causal_and_bounded():
    cfg = dict(vocab_size=50, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=8, rope_theta=100.0, sliding_window=4, attn_logit_softcapping=5.0,
               final_logit_softcapping=3.0, query_pre_attn_scalar=8, rms_norm_eps=1e-6)
    g = torch.Generator().manual_seed(2)
    w = {"model.embed_tokens.weight": torch.randn(50, 32, generator=g), "model.norm.weight": torch.randn(32, generator=g) * 0.1}
    for i in range(2):
        p = f"model.layers.{i}."
        for n, shape in (("self_attn.q_proj", (32, 32)), ("self_attn.k_proj", (16, 32)), ("self_attn.v_proj", (16, 32)),
                         ("self_attn.o_proj", (32, 32)), ("mlp.gate_proj", (48, 32)), ("mlp.up_proj", (48, 32)),
                         ("mlp.down_proj", (32, 48))):
            w[p + n + ".weight"] = torch.randn(shape, generator=g) * 0.3
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            w[p + n + ".weight"] = torch.randn(32, generator=g) * 0.1
    ids = [3, 14, 15, 9, 2, 6, 5, 35]
    out = plain.forward(cfg, w, ids)
    assert out.shape == (8, 50) and float(out.abs().max()) <= 3.0
    assert torch.allclose(plain.forward(cfg, w, ids[:5]), out[:5])               # a prefix gives the same logits
    assert plain.layer_is_sliding(cfg, 0) and not plain.layer_is_sliding(cfg, 1)
    assert plain.layer_is_sliding({**cfg, "layer_types": ["full_attention", "sliding_attention"]}, 1)
    gen = plain.greedy(cfg, w, ids[:3], 4)
    assert len(gen) == 4 and gen[0] == int(torch.argmax(plain.forward(cfg, w, ids[:3])[-1]))
    assert plain.greedy(cfg, w, ids[:3], 4, stop_ids=(gen[2],)) == gen[:gen.index(gen[2])]


def test_sampler_oracle():
    logits = torch.tensor([1.0, 3.0, 2.0, -1.0, 2.0])
    assert sampling_plain.sample(logits, 0.0, 0, 1.0, 0.3) == 1 and sampling_plain.sample(logits, 1.0, 1, 1.0, 0.9) == 1
    probs, mask = sampling_plain.kept_set(logits, 1.0, 2, 1.0)
    assert mask.tolist() == [False, True, True, False, True]                    # the tie with the second one is kept
    probs, mask = sampling_plain.kept_set(logits, 1.0, 0, 0.5)
    assert mask.tolist() == [False, True, False, False, False]                  # p(1) = 0.53 already reaches 0.5
    probs, mask = sampling_plain.kept_set(logits, 1.0, 0, 1.0)
    draws = [sampling_plain.sample(logits, 1.0, 0, 1.0, u) for u in (0.0, 0.05, 0.5, 0.99)]
    cdf = torch.cumsum(probs, 0)
    assert draws == [int((cdf > u).nonzero()[0]) for u in (0.0, 0.05, 0.5, 0.99)]


def test_two_independent_restatements_agree(tmp_path):
    """The whole-sequence oracle (torch, masks over matrices) and the token-by-token one (NumPy, lists of
    keys and values, complex rotation) were written apart from each other from the same lines of
    wlejon/brolm; they must give the same logits, prompts longer than the window included.  The
    window's edge in particular: both keep exactly ``sliding_window`` keys, the query's own included."""
    import numpy as np

    from tests.helpers import TINY, make_folder, oracle_inputs, random_prompts
    from tests.plain import gemma2_stepwise as stepwise
    for name in TINY:
        folder = make_folder(tmp_path, name, torch.float32)
        config, weights = oracle_inputs(folder)
        W = config["sliding_window"]
        for p in random_prompts(config["vocab_size"], [1, W, W + 1, 2 * W + 7], seed=3):
            a = plain.forward(config, weights, p).numpy()
            b = stepwise.forward(config, weights, p)
            assert a.shape == b.shape
            assert float(np.abs(a - b).max()) <= 1e-9 * max(1.0, float(np.abs(a).max())), (name, len(p))
    # the edge itself: with window W the logits at position W do not depend on token 0, at W - 1 they do
    config, weights = oracle_inputs(make_folder(tmp_path, "A", torch.float32))
    config = {**config, "layer_types": ["sliding_attention"] * config["num_hidden_layers"]}
    W = config["sliding_window"]
    p = random_prompts(config["vocab_size"], [W + 1], seed=4)[0]
    q = [(p[0] + 1) % config["vocab_size"]] + p[1:]
    for impl in (lambda ids: plain.forward(config, weights, ids).numpy(), lambda ids: stepwise.forward(config, weights, ids)):
        x, y = impl(p), impl(q)
        # every layer slides: position W sees keys 1..W only, and those keys were made from positions that
        # themselves saw token 0 at most through W - 1 earlier keys ... in a model of one layer; with more
        # layers token 0 reaches further, so the statement is checked on the first layer's reach only
        assert float(np.abs(x[W - 1] - y[W - 1]).max()) > 1e-6
    one = {**config, "num_hidden_layers": 1, "layer_types": ["sliding_attention"]}
    for impl in (lambda ids: plain.forward(one, weights, ids).numpy(), lambda ids: stepwise.forward(one, weights, ids)):
        x, y = impl(p), impl(q)
        assert float(np.abs(x[W] - y[W]).max()) == 0.0 and float(np.abs(x[W - 1] - y[W - 1]).max()) > 1e-6
