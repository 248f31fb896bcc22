"""Plain, slow restatement of the Gemma 2 decoder used as the oracle of the tests.

Whole sequences, no cache, one function per part, float64 on the CPU.  It
shares no code with ``brolm_b200``: it reads ``config.json`` as a plain dict
and the weights as a plain ``{name: tensor}`` dict.

It rests on the formulas of wlejon/brolm's C++ sources, not on a run of them:
brolm's model code needs the sibling library brotensor (``CMakeLists.txt:64-76``
stops with FATAL_ERROR without it), which is not part of the reference tree,
so ``src/gemma2.cpp`` cannot be compiled here.  Every function below cites the
lines it restates (paths are relative to the brolm project root).

Two places deliberately follow the checkpoint rather than brolm's device
layout, with equal results:

* RoPE pairs element ``i`` with ``i + head_dim/2`` (the layout of the stored
  q/k projections).  brolm permutes the rows of Wq/Wk at load
  (``include/brolm/detail/weights.h:106-127``) and then rotates adjacent pairs
  (``src/gemma2.cpp:355-356``); a common permutation inside each head of q and
  k leaves every score q.k unchanged.
* The score scale is ``query_pre_attn_scalar ** -0.5``.  brolm uses the
  attention op's built-in ``head_dim ** -0.5`` and refuses configurations in
  which the two differ (``src/gemma2_config.cpp:200-209``).
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def layer_is_sliding(config: dict, layer: int) -> bool:
    """Even layers slide, odd layers are global (src/gemma2.cpp:364).

    An explicit ``layer_types`` list in config.json wins when it is present.
    """
    kinds = config.get("layer_types")
    if kinds:
        return kinds[layer] == "sliding_attention"
    return layer % 2 == 0


def embed(table: torch.Tensor, ids: torch.Tensor, hidden: int) -> torch.Tensor:
    """h[t] = E[ids[t]] * sqrt(hidden)  (src/gemma2.cpp:283-285, 340-343).

    The scale is the float32 value of sqrt(hidden), as in the reference.
    """
    scale = float(torch.tensor(float(hidden), dtype=torch.float32).sqrt())
    return table.to(DT)[ids.long()] * scale


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * (1 + w)

    (src/gemma2.cpp:154-175 folds the +1 into the gain; :349 applies it).
    """
    x = x.to(DT)
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inv * (1.0 + w.to(DT))


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Y = X W^T, W stored (out, in), no bias (include/brolm/detail/compute.h:49-86)."""
    return x.to(DT) @ w.to(DT).t()


def rope(x: torch.Tensor, positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """Rotate each head of x (T, heads*head_dim) by its token's position.

    Frequency i in [0, head_dim/2) is theta ** (-2 i / head_dim)
    (schedule as brolm states it, src/qwen35_text.cpp:220-256); the pair is
    (i, i + head_dim/2) (see the module docstring); positions are absolute
    (src/gemma2.cpp:336-338).
    """
    T = x.shape[0]
    half = head_dim // 2
    xh = x.to(DT).reshape(T, -1, head_dim)
    i = torch.arange(half, dtype=DT)
    inv_freq = torch.tensor(theta, dtype=DT) ** (-2.0 * i / head_dim)
    ang = positions.to(DT)[:, None] * inv_freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = xh[..., :half], xh[..., half:]
    out = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
    return out.reshape(T, -1)


def soft_cap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """cap * tanh(x / cap) when cap > 0 (src/gemma2.cpp:406-412)."""
    if cap and cap > 0:
        return cap * torch.tanh(x / cap)
    return x


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_q: int, n_kv: int,
              head_dim: int, scale: float, cap: float, window: int) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    q (T, n_q*hd), k and v (T, n_kv*hd), all after RoPE where it applies.
    Query head h reads kv head h // (n_q // n_kv)
    (src/detail/dense_decoder.cpp:593-594).  Scores are scaled, soft-capped,
    masked, then softmaxed (src/gemma2.cpp:360-367).  ``window`` 0 means
    global; otherwise key j is visible from query p iff 0 <= p - j < window.
    """
    T = q.shape[0]
    group = n_q // n_kv
    qh = q.to(DT).reshape(T, n_q, head_dim)
    kh = k.to(DT).reshape(T, n_kv, head_dim)
    vh = v.to(DT).reshape(T, n_kv, head_dim)
    out = torch.zeros(T, n_q, head_dim, dtype=DT)
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    visible = dist >= 0
    if window and window > 0:
        visible = visible & (dist < window)
    for h in range(n_q):
        g = h // group
        s = (qh[:, h, :] @ kh[:, g, :].t()) * scale
        s = soft_cap(s, cap)
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ vh[:, g, :]
    return out.reshape(T, n_q * head_dim)


def attention_last_query(q_row: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_q: int, n_kv: int,
                         head_dim: int, scale: float, cap: float, window: int) -> torch.Tensor:
    """The last row of ``attention`` alone: one query (n_q*hd,) at position T - 1 over keys 0 .. T - 1.

    What a decode step computes (src/gemma2.cpp:365-367 with L = 1); the same formulas, for tests
    whose sequences are too long for a T x T matrix per head.
    """
    T = k.shape[0]
    group = n_q // n_kv
    qh = q_row.to(DT).reshape(n_q, head_dim)
    kh = k.to(DT).reshape(T, n_kv, head_dim)
    vh = v.to(DT).reshape(T, n_kv, head_dim)
    first = max(0, T - window) if window and window > 0 else 0          # 0 <= (T - 1) - j < window
    out = torch.zeros(n_q, head_dim, dtype=DT)
    for h in range(n_q):
        g = h // group
        s = soft_cap((kh[first:, g, :] @ qh[h]) * scale, cap)
        out[h] = torch.softmax(s, dim=0) @ vh[first:, g, :]
    return out.reshape(n_q * head_dim)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    """0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))  (src/gemma2.cpp:380)."""
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def feed_forward(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """down(gelu_tanh(gate(x)) * up(x))  (src/gemma2.cpp:378-382)."""
    return linear(gelu_tanh(linear(x, wg)) * linear(x, wu), wd)


def decoder_layer(h: torch.Tensor, w: dict, prefix: str, config: dict, layer: int) -> torch.Tensor:
    """One layer with its four norms (src/gemma2.cpp:345-387)."""
    eps = config["rms_norm_eps"]
    hd = config["head_dim"]
    n_q, n_kv = config["num_attention_heads"], config["num_key_value_heads"]
    T = h.shape[0]
    positions = torch.arange(T)

    x = rms_norm(h, w[prefix + "input_layernorm.weight"], eps)
    q = rope(linear(x, w[prefix + "self_attn.q_proj.weight"]), positions, hd, config["rope_theta"])
    k = rope(linear(x, w[prefix + "self_attn.k_proj.weight"]), positions, hd, config["rope_theta"])
    v = linear(x, w[prefix + "self_attn.v_proj.weight"])
    window = config["sliding_window"] if layer_is_sliding(config, layer) else 0
    a = attention(q, k, v, n_q, n_kv, hd, float(config["query_pre_attn_scalar"]) ** -0.5,
                  config.get("attn_logit_softcapping") or 0.0, window)
    y = linear(a, w[prefix + "self_attn.o_proj.weight"])
    h = h + rms_norm(y, w[prefix + "post_attention_layernorm.weight"], eps)

    x = rms_norm(h, w[prefix + "pre_feedforward_layernorm.weight"], eps)
    y = feed_forward(x, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                     w[prefix + "mlp.down_proj.weight"])
    return h + rms_norm(y, w[prefix + "post_feedforward_layernorm.weight"], eps)


def hidden(config: dict, w: dict, ids) -> torch.Tensor:
    """The rows the output matrix is given, (T, hidden): the residual stream after the final norm,
    what the reference hands out as ``hidden_out`` (src/gemma2.cpp:389-391)."""
    ids = torch.as_tensor(ids)
    h = embed(w["model.embed_tokens.weight"], ids, config["hidden_size"])
    for i in range(config["num_hidden_layers"]):
        h = decoder_layer(h, w, f"model.layers.{i}.", config, i)
    return rms_norm(h, w["model.norm.weight"], config["rms_norm_eps"])


def forward(config: dict, w: dict, ids) -> torch.Tensor:
    """Logits (T, vocab) of one whole sequence (src/gemma2.cpp:272-288, 326-415)."""
    x = hidden(config, w, ids)
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])  # src/gemma2.cpp:223-234
    return soft_cap(linear(x, head), config.get("final_logit_softcapping") or 0.0)


def greedy(config: dict, w: dict, prompt, max_new: int, stop_ids=()) -> list[int]:
    """Greedy continuation by full recomputation (include/brolm/detail/generate.h:78-123).

    A stop token ends the sequence and is not returned (generate.h:106-118).
    """
    ids = list(prompt)
    out: list[int] = []
    if not ids or max_new <= 0:
        return out
    while len(out) < max_new:
        nxt = int(torch.argmax(forward(config, w, ids)[-1]))  # first maximum wins (src/detail/generate.cpp:38-48)
        if nxt in stop_ids:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
