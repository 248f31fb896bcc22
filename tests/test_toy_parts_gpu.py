"""A new mixer with state of its own, a new architecture and an unusual
schedule, all defined here and run through the unchanged framework: the toy
is registered, built from a config.json, loaded from safetensors, and stepped
(prompt, decode, unequal batch, reused slots) against its own plain formula."""
import dataclasses
import json
import os
from typing import ClassVar

import pytest
import torch

import brolm_b200 as bb
from brolm_b200.cache import StateSpec
from brolm_b200.parts import (BlockSpec, EmbeddingSpec, HeadSpec, LayerCall, ModelLayout, ParamSpec, Part, PartSpec,
                              linear)
from tests.plain import gemma2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class DecayMixer(Part):
    """y_t = W s_t with s_t = decay * s_{t-1} + x_t: a running state per sequence, no keys."""
    kind = "mixer"

    def __init__(self, hidden: int, decay: float):
        self.hidden, self.decay = hidden, decay

    def param_specs(self):
        return {"w": ParamSpec((self.hidden, self.hidden))}

    def cache_spec(self):
        return StateSpec((self.hidden,), torch.float32)

    def forward(self, x, ctx, entry, writes_cache=True):
        state = ctx.state(entry)                      # [max_slots, hidden] float32
        slots = ctx.slots_dev.long()
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        cu = ctx.cu_q.tolist()
        for b in range(ctx.batch):
            s = state[slots[b]].clone()
            for t in range(cu[b], cu[b + 1]):
                s = self.decay * s + x[t].float()
                out[t] = s
            state[slots[b]] = s
        return linear(out.to(ctx.dtype), self.params["w"], out_dtype=torch.float32)


bb.register_part("mixer", "toy_decay", DecayMixer)


@dataclasses.dataclass
class ToyConfig(bb.ModelConfig):
    architecture: ClassVar[str] = "ToyDecayForCausalLM"
    model_types: ClassVar[tuple] = ("toy_decay",)
    vocab_size: int = 120
    hidden_size: int = 48
    inter: int = 80
    decay: float = 0.5
    eps: float = 1e-5

    def validate(self):
        if self.hidden_size % 16:
            raise bb.ConfigError("ToyConfig: hidden_size must be a multiple of 16")


def toy_layout(cfg: ToyConfig) -> ModelLayout:
    H = cfg.hidden_size

    def norm(name):
        return PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.eps, offset=0.0), {"weight": name})

    def ffn(i):
        return PartSpec("feedforward", "gated", dict(hidden=H, inter=cfg.inter, activation="silu"),
                        {"gate": f"l{i}.gate", "up": f"l{i}.up", "down": f"l{i}.down"})

    decay = PartSpec("mixer", "toy_decay", dict(hidden=H, decay=cfg.decay), {"w": "l0.mix"})
    attn = PartSpec("mixer", "attention", dict(hidden=H, n_q=3, n_kv=1, head_dim=16, scale=0.25, softcap=0.0,
                                               window=None, position=PartSpec("position", "rope",
                                                                              dict(head_dim=16, theta=100.0))),
                    {"q": "l1.q", "k": "l1.k", "v": "l1.v", "o": "l1.o"})
    blocks = [BlockSpec(decay, ffn(0), norm("l0.n1"), norm("l0.n2")),                  # pre-norm only
              BlockSpec(attn, ffn(1), norm("l1.n1"), norm("l1.n2"), norm("l1.n3"), norm("l1.n4"))]
    # block 0 runs twice (each run keeps a state of its own); the last call reads call 1's keys
    schedule = [LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache_of=1)]
    return ModelLayout(EmbeddingSpec("emb", cfg.vocab_size, H, 1.0), blocks, schedule, norm("final"),
                       HeadSpec("head", tied_to=None, softcap=0.0), weight_std=0.1, norm_std=0.1)


bb.register_architecture(ToyConfig, toy_layout)


def toy_oracle(cfg, w, ids):
    """Whole sequence, float64, from the formulas above."""
    D = torch.float64
    h = w["emb"].to(D)[torch.tensor(ids)]
    T = len(ids)
    pos = torch.arange(T)

    def nrm(x, name):
        return plain.rms_norm(x, w[name] - 1.0, cfg.eps)      # offset 0: gain is w itself

    def ffn(x, i):
        g = plain.linear(x, w[f"l{i}.gate"])
        return plain.linear(g * torch.sigmoid(g) * plain.linear(x, w[f"l{i}.up"]), w[f"l{i}.down"])

    def decay_block(h):
        x = nrm(h, "l0.n1")
        s = torch.zeros(cfg.hidden_size, dtype=D)
        out = []
        for t in range(T):
            s = cfg.decay * s + x[t]
            out.append(s)
        h = h + plain.linear(torch.stack(out), w["l0.mix"])
        return h + ffn(nrm(h, "l0.n2"), 0)

    kv = {}

    def attn_block(h, reuse):
        x = nrm(h, "l1.n1")
        q = plain.rope(plain.linear(x, w["l1.q"]), pos, 16, 100.0)
        if not reuse:
            kv["k"] = plain.rope(plain.linear(x, w["l1.k"]), pos, 16, 100.0)
            kv["v"] = plain.linear(x, w["l1.v"])
        a = plain.attention(q, kv["k"], kv["v"], 3, 1, 16, 0.25, 0.0, 0)
        h = h + nrm(plain.linear(a, w["l1.o"]), "l1.n3")
        return h + nrm(ffn(nrm(h, "l1.n2"), 1), "l1.n4")

    h = decay_block(h)
    h = attn_block(h, False)
    h = decay_block(h)
    h = attn_block(h, True)
    return plain.linear(nrm(h, "final"), w["head"])


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_toy_architecture_runs_through_the_unchanged_framework(tmp_path, dtype, tol):
    cfg = ToyConfig()
    folder = str(tmp_path / "toy")
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    bb.write_random_model(cfg, folder, seed=3, dtype=store)
    with open(os.path.join(folder, "config.json")) as fh:
        assert json.load(fh)["architectures"] == ["ToyDecayForCausalLM"]
    from safetensors.torch import load_file
    w = load_file(os.path.join(folder, "model.safetensors"))
    model = bb.load_model(folder, dtype=dtype, device=DEV)
    assert isinstance(model.config, ToyConfig)
    eng = bb.Engine(model, max_tokens=512, max_slots=3)
    assert len(eng.cache.state_groups) == 1 and len(eng.cache.state_groups[0].entries) == 2
    assert len(eng.cache.kv_groups) == 1 and len(eng.cache.kv_groups[0].entries) == 1

    g = torch.Generator().manual_seed(4)
    for round_ in range(2):                      # the second round reuses slots whose state must start at zero
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (30, 7, 70)]
        refs = [toy_oracle(cfg, w, p) for p in prompts]
        pre = [20, 1, 66]
        slots = eng.open(3)
        got = eng.step(slots, [p[:k] for p, k in zip(prompts, pre)], want=[list(range(k)) for k in pre])
        off = 0
        for r, k in zip(refs, pre):
            assert float((got[off:off + k].double().cpu() - r[:k]).abs().max()) <= tol
            off += k
        done = list(pre)
        live = [0, 1, 2]
        while live:
            got = eng.step([slots[i] for i in live], [[prompts[i][done[i]]] for i in live])
            for row, i in enumerate(live):
                assert float((got[row].double().cpu() - refs[i][done[i]]).abs().max()) <= tol
                done[i] += 1
            live = [i for i in live if done[i] < len(prompts[i])]
        eng.close(slots)
