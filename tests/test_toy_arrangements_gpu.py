"""Three more things a new architecture may bring, defined here and run through the
unchanged framework:

* a norm that is not an RMSNorm (mean-subtracting, with a bias): the residual sum stays fused,
  the norm runs through its own ``apply``, before and after the sum, also when the sublayer's
  output arrives as partial sums of a product cut along K;
* another arrangement of a layer's parts, registered as a ``block``: mixer and feed-forward
  read the same normed input and both add to the residual stream (a "parallel" block);
* a mixer with state of its own whose decode step reads nothing back to the host, so the step is
  captured in a CUDA graph: padding rows of a captured batch must leave every live sequence's
  state alone (three sequences run in a graph of four rows, slot 0 among them).
"""
import dataclasses
from typing import ClassVar

import pytest
import torch

import brolm_b200 as bb
from brolm_b200.cache import StateSpec
from brolm_b200.parts import (BlockSpec, EmbeddingSpec, HeadSpec, LayerCall, ModelLayout, ParamSpec, Part, PartSpec,
                              add_then_norm, linear)
from tests.plain import gemma2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class ToyLayerNorm(Part):
    """y = (x - mean) / sqrt(var + eps) * (1 + w) + b, in float32."""
    kind = "norm"
    graph_safe = True

    def __init__(self, size: int, eps: float):
        self.size, self.eps = size, eps

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), "vector"), "bias": ParamSpec((self.size,), "vector")}

    def apply(self, x, out_dtype, rows=None):
        if rows is not None:
            x = x.index_select(0, rows.long())
        x = x.float()
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        y = (x - mu) * torch.rsqrt(var + self.eps) * (1.0 + self.params["weight"].float()) + self.params["bias"].float()
        return y.to(out_dtype)


class RunningSum(Part):
    """y_t = W s_t with s_t = decay * s_{t-1} + x_t, written with device operations only."""
    kind = "mixer"
    graph_safe = True

    def __init__(self, hidden: int, decay: float):
        self.hidden, self.decay = hidden, decay

    def param_specs(self):
        return {"w": ParamSpec((self.hidden, self.hidden))}

    def cache_spec(self):
        return StateSpec((self.hidden,), torch.float32)

    def forward(self, x, ctx, entry, writes_cache=True):
        state = ctx.state(entry)                      # [max_slots + 1, hidden] float32
        slots = ctx.slots_dev.long()
        xf = x.float()
        if ctx.mode == "decode":
            s = self.decay * state.index_select(0, slots) + xf
            state.index_copy_(0, slots, s)            # padding rows all write the spare row
            out = s
        else:
            # every sequence starts from a zero state: s_t = sum over j <= t of its own tokens decay^(t-j) x_j
            pos, seq = ctx.positions.long(), ctx.tok_seq.long()
            dist = pos[:, None] - pos[None, :]
            mine = (seq[:, None] == seq[None, :]) & (dist >= 0)
            weight = torch.where(mine, torch.pow(torch.tensor(self.decay, device=x.device), dist.clamp(min=0).float()),
                                 torch.zeros((), device=x.device))
            out = weight @ xf
            last = ctx.cu_q[1:].long() - 1
            state.index_copy_(0, slots, out.index_select(0, last))
        return linear(out.to(ctx.dtype), self.params["w"], out_dtype=torch.float32)


class ParallelBlock(Part):
    """x = norm(h);  h += mixer(x) + feedforward(x)."""
    kind = "block"

    def __init__(self, mixer, feedforward, norm):
        self.mixer, self.feedforward, self.norm = mixer, feedforward, norm

    def parts(self):
        return {"mixer": self.mixer, "feedforward": self.feedforward, "norm": self.norm}

    @property
    def entry_norm(self):
        return self.norm

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, h, x, ctx, entry, writes_cache, next_norm):
        a = self.mixer.forward(x, ctx, entry, writes_cache)
        b = self.feedforward.forward(x, ctx)
        add_then_norm(h, a, None, None, ctx.dtype)
        return add_then_norm(h, b, None, next_norm, ctx.dtype)


bb.register_part("norm", "toy_layernorm", ToyLayerNorm)
bb.register_part("mixer", "toy_running_sum", RunningSum)
bb.register_part("block", "toy_parallel", ParallelBlock)

N_Q, N_KV, HD = 8, 2, 256          # a wide attention output: its projection back is cut along K in a decode step


@dataclasses.dataclass
class ToyParConfig(bb.ModelConfig):
    architecture: ClassVar[str] = "ToyParallelForCausalLM"
    model_types: ClassVar[tuple] = ("toy_parallel",)
    vocab_size: int = 90
    hidden_size: int = 32
    inter: int = 48
    decay: float = 0.75
    eps: float = 1e-5


def toy_par_layout(cfg: ToyParConfig) -> ModelLayout:
    H = cfg.hidden_size

    def ln(name):
        return PartSpec("norm", "toy_layernorm", dict(size=H, eps=cfg.eps), {"weight": name + ".w", "bias": name + ".b"})

    def rms(name):
        return PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.eps, offset=1.0), {"weight": name})

    def ffn(i):
        return PartSpec("feedforward", "gated", dict(hidden=H, inter=cfg.inter, activation="gelu_tanh"),
                        {"gate": f"l{i}.gate", "up": f"l{i}.up", "down": f"l{i}.down"})

    run = PartSpec("mixer", "toy_running_sum", dict(hidden=H, decay=cfg.decay), {"w": "l0.mix"})
    attn = PartSpec("mixer", "attention", dict(hidden=H, n_q=N_Q, n_kv=N_KV, head_dim=HD, scale=HD ** -0.5, softcap=0.0,
                                               window=None, position=PartSpec("position", "rope",
                                                                              dict(head_dim=HD, theta=100.0))),
                    {"q": "l1.q", "k": "l1.k", "v": "l1.v", "o": "l1.o"})
    blocks = [BlockSpec(kind="toy_parallel", mixer=run, feedforward=ffn(0), more={"norm": ln("l0.n")}),
              # a layer norm before the mixer (the block before cannot fuse it), one after the mixer (it gets the
              # product's partial sums), RMSNorms around the feed-forward (fused with the sums)
              BlockSpec(attn, ffn(1), pre_mixer_norm=ln("l1.n1"), pre_ffn_norm=rms("l1.n2"),
                        post_mixer_norm=ln("l1.n3"), post_ffn_norm=rms("l1.n4"))]
    schedule = [LayerCall(0), LayerCall(1), LayerCall(0)]
    return ModelLayout(EmbeddingSpec("emb", cfg.vocab_size, H, 1.0), blocks, schedule, ln("final"),
                       HeadSpec("head", tied_to=None, softcap=0.0), weight_std=0.1, norm_std=0.1)


bb.register_architecture(ToyParConfig, toy_par_layout)


def oracle(cfg, w, ids):
    D = torch.float64
    T = len(ids)
    pos = torch.arange(T)
    h = w["emb"].to(D)[torch.tensor(ids)]

    def ln(x, name):
        x = x.to(D)
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        return (x - mu) / torch.sqrt(var + cfg.eps) * (1.0 + w[name + ".w"].to(D)) + w[name + ".b"].to(D)

    def ffn(x, i):
        return plain.feed_forward(x, w[f"l{i}.gate"], w[f"l{i}.up"], w[f"l{i}.down"])

    def parallel(h):
        x = ln(h, "l0.n")
        s = torch.zeros(cfg.hidden_size, dtype=D)
        out = []
        for t in range(T):
            s = cfg.decay * s + x[t]
            out.append(s)
        return h + plain.linear(torch.stack(out), w["l0.mix"]) + ffn(x, 0)

    def sandwich(h):
        x = ln(h, "l1.n1")
        q = plain.rope(plain.linear(x, w["l1.q"]), pos, HD, 100.0)
        k = plain.rope(plain.linear(x, w["l1.k"]), pos, HD, 100.0)
        a = plain.attention(q, k, plain.linear(x, w["l1.v"]), N_Q, N_KV, HD, HD ** -0.5, 0.0, 0)
        h = h + ln(plain.linear(a, w["l1.o"]), "l1.n3")
        return h + plain.rms_norm(ffn(plain.rms_norm(h, w["l1.n2"], cfg.eps), 1), w["l1.n4"], cfg.eps)

    return plain.linear(ln(parallel(sandwich(parallel(h))), "final"), w["head"])


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_other_norm_other_arrangement_and_a_captured_state_mixer(tmp_path, dtype, tol):
    from brolm_b200 import kernels
    from safetensors.torch import load_file
    cfg = ToyParConfig()
    folder = str(tmp_path / "toy")
    bb.write_random_model(cfg, folder, seed=5, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    w = load_file(f"{folder}/model.safetensors")
    model = bb.load_model(folder, dtype=dtype, device=DEV)
    assert type(model.blocks[0]).__name__ == "ParallelBlock" and type(model.final_norm).__name__ == "ToyLayerNorm"
    eng = bb.Engine(model, max_tokens=512, max_slots=4)
    assert eng.use_graphs                          # every part says it is graph safe
    if dtype == "bfloat16":
        # the case the unfused norm must handle: the product before it comes in slices of K
        x = torch.zeros(3, N_Q * HD, dtype=torch.bfloat16, device=DEV)
        assert kernels.skinny_parts(x, model.blocks[1].mixer.w_o) > 1
    g = torch.Generator().manual_seed(6)
    for round_ in range(2):
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (30, 12, 70)]
        refs = [oracle(cfg, w, p) for p in prompts]
        pre = [20, 1, 66]
        slots = eng.open(3)
        assert 0 in slots                          # slot 0 is live while a padding row exists
        got = eng.step(slots, [p[:k] for p, k in zip(prompts, pre)], want=[list(range(k)) for k in pre])
        off = 0
        for r, k in zip(refs, pre):
            assert float((got[off:off + k].double().cpu() - r[:k]).abs().max()) <= tol
            off += k
        done = list(pre)
        live = [0, 1, 2]
        while live:
            # three rows run in a captured step of four: the fourth is padding
            got = eng.step([slots[i] for i in live], [[prompts[i][done[i]]] for i in live])
            for row, i in enumerate(live):
                assert float((got[row].double().cpu() - refs[i][done[i]]).abs().max()) <= tol, (round_, i, done[i])
                done[i] += 1
            live = [i for i in live if done[i] < len(prompts[i])]
        eng.close(slots)
    assert any(g.rows == 4 for g in eng._graphs.values())
