"""A second plain restatement of the Gemma 2 decoder, independent of ``gemma2_plain``.

NumPy, float64, one token at a time: every layer keeps a Python list of the
keys and values it has seen, a new token is pushed through all layers against
those lists, and its logits come out before the next token goes in.  It was
written from wlejon/brolm's ``Gemma2Model::run_layers_`` (src/gemma2.cpp:326-415)
read as a decode step (L = 1 at cache length P, the form :336-338 and :365
describe), not from the whole-sequence oracle next to it, and it shares no
code with that oracle or with ``brolm_b200``.  Where the two restatements could
disagree they are built differently on purpose:

* the rotation is a complex product ``(a + i b) * exp(i * phi)`` over the pair
  (a, b) = (x[i], x[i + head_dim/2]) instead of two real formulas;
* the window is stated on the list of keys, "the newest ``window`` entries, the
  token's own included", instead of a mask over a distance matrix;
* the softmax is written out with an explicit maximum and sum;
* norms divide by a square root instead of multiplying by ``rsqrt``.

A test requires both to give the same logits to 1e-9; the engine is compared
with ``gemma2_plain``.  Like that one it rests on the formulas, not on a run of
brolm (src/gemma2.cpp does not build without the absent brotensor).
"""
from __future__ import annotations

import math

import numpy as np


def _f64(t) -> np.ndarray:
    """A checkpoint tensor (torch, any float type) as float64."""
    if hasattr(t, "detach"):
        t = t.detach().to("cpu").double().numpy()
    return np.asarray(t, dtype=np.float64)


class StepwiseGemma2:
    """One sequence, token by token.  ``push(token)`` returns that token's logits."""

    def __init__(self, config: dict, weights: dict):
        self.c = config
        self.w = {k: _f64(v) for k, v in weights.items()}
        self.n_layers = int(config["num_hidden_layers"])
        self.keys = [[] for _ in range(self.n_layers)]       # per layer: one (n_kv, head_dim) array per token
        self.values = [[] for _ in range(self.n_layers)]
        self.position = 0

    # parts ----------------------------------------------------------------
    def norm(self, x: np.ndarray, gain: np.ndarray) -> np.ndarray:
        # rms_norm_forward with the +1 that load_weights folds into the gain (src/gemma2.cpp:154-175, :349)
        rms = math.sqrt(float(np.dot(x, x)) / x.size + float(self.c["rms_norm_eps"]))
        return (x / rms) * (gain + 1.0)

    def rotate(self, heads: np.ndarray, position: int) -> np.ndarray:
        # rope_forward at the token's absolute position (src/gemma2.cpp:336-338, :355-356); the pair of
        # frequency i is (i, i + head_dim/2), the order the checkpoint stores (include/brolm/gemma2.h:38-40)
        hd = heads.shape[-1]
        half = hd // 2
        freq = float(self.c["rope_theta"]) ** (-np.arange(half, dtype=np.float64) * 2.0 / hd)
        turn = np.exp(1j * position * freq)
        z = (heads[:, :half] + 1j * heads[:, half:]) * turn[None, :]
        return np.concatenate([z.real, z.imag], axis=1)

    def sliding(self, layer: int) -> bool:
        kinds = self.c.get("layer_types")
        if kinds:
            return kinds[layer] == "sliding_attention"
        return layer % 2 == 0                                   # src/gemma2.cpp:364

    def attend(self, layer: int, q: np.ndarray) -> np.ndarray:
        # flash_attention_decode over the cache with the soft-cap and the window (src/gemma2.cpp:360-367)
        c = self.c
        n_q, n_kv = int(c["num_attention_heads"]), int(c["num_key_value_heads"])
        keys, values = self.keys[layer], self.values[layer]
        if self.sliding(layer):
            w = int(c["sliding_window"])
            keys, values = keys[-w:], values[-w:]               # the newest w entries, this token's included
        scale = 1.0 / math.sqrt(float(c["query_pre_attn_scalar"]))
        cap = float(c.get("attn_logit_softcapping") or 0.0)
        out = np.zeros_like(q)
        for h in range(n_q):
            g = h // (n_q // n_kv)
            scores = np.array([float(np.dot(q[h], k[g])) * scale for k in keys])
            if cap > 0.0:
                scores = cap * np.tanh(scores / cap)
            e = np.exp(scores - scores.max())
            p = e / e.sum()
            for pj, v in zip(p, values):
                out[h] += pj * v[g]
        return out

    def feed_forward(self, x: np.ndarray, prefix: str) -> np.ndarray:
        # gate, up, gelu (tanh form), product, down (src/gemma2.cpp:378-382)
        w = self.w
        gate = w[prefix + "mlp.gate_proj.weight"] @ x
        up = w[prefix + "mlp.up_proj.weight"] @ x
        act = 0.5 * gate * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (gate + 0.044715 * gate * gate * gate)))
        return w[prefix + "mlp.down_proj.weight"] @ (act * up)

    # the step -------------------------------------------------------------
    def push(self, token: int) -> np.ndarray:
        c, w = self.c, self.w
        hd = int(c["head_dim"])
        n_q, n_kv = int(c["num_attention_heads"]), int(c["num_key_value_heads"])
        p = self.position
        # embedding row times the float32 value of sqrt(hidden) (src/gemma2.cpp:283-285, :340-343)
        h = w["model.embed_tokens.weight"][int(token)] * float(np.sqrt(np.float32(c["hidden_size"])))
        for layer in range(self.n_layers):
            pre = f"model.layers.{layer}."
            x = self.norm(h, w[pre + "input_layernorm.weight"])
            q = self.rotate((w[pre + "self_attn.q_proj.weight"] @ x).reshape(n_q, hd), p)
            k = self.rotate((w[pre + "self_attn.k_proj.weight"] @ x).reshape(n_kv, hd), p)
            v = (w[pre + "self_attn.v_proj.weight"] @ x).reshape(n_kv, hd)
            self.keys[layer].append(k)                         # kv_cache_append (src/gemma2.cpp:358)
            self.values[layer].append(v)
            a = self.attend(layer, q).reshape(n_q * hd)
            y = w[pre + "self_attn.o_proj.weight"] @ a
            h = h + self.norm(y, w[pre + "post_attention_layernorm.weight"])          # :371-373
            x = self.norm(h, w[pre + "pre_feedforward_layernorm.weight"])
            y = self.feed_forward(x, pre)
            h = h + self.norm(y, w[pre + "post_feedforward_layernorm.weight"])        # :384-386
        x = self.norm(h, w["model.norm.weight"])
        head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]   # :223-234
        logits = head @ x
        cap = float(c.get("final_logit_softcapping") or 0.0)
        if cap > 0.0:
            logits = cap * np.tanh(logits / cap)               # :406-412
        self.position += 1
        return logits


def forward(config: dict, weights: dict, ids) -> np.ndarray:
    """Logits (T, vocab) of one sequence, computed token by token."""
    model = StepwiseGemma2(config, weights)
    return np.stack([model.push(int(t)) for t in ids])
