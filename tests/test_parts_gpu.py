"""Each part of a layer alone (norm, position encoding, attention mixer,
feed-forward, the block's arrangement) against the plain formulas."""
import math

import pytest
import torch

import brolm_b200 as bb
from brolm_b200.parts import Attention, Block, GatedFeedForward, RMSNorm, RotaryEmbedding
from brolm_b200.cache import Cache
from brolm_b200.engine.context import StepContext
from tests.plain import gemma2_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def rel(got, ref):
    ref = ref.double().cpu()
    return float((got.double().cpu() - ref).abs().max()) / max(1e-30, float(ref.abs().max()))


def make_ctx(cache, mode, lengths_before, n_new, dtype):
    """A step context by hand, for parts used outside a model."""
    B = len(n_new)
    slots = [cache.alloc_slot() for _ in range(B)] if mode == "prefill" else list(range(B))
    new_len = [a + b for a, b in zip(lengths_before, n_new)]
    cache.reserve(dict(zip(slots, new_len)))
    cache.commit(dict(zip(slots, new_len)))
    cu = [0]
    for n in n_new:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return StepContext(
        mode=mode, dtype=dtype, device=DEV, cache=cache, batch=B, n_tokens=cu[-1], slots=slots,
        positions=i32([p for a, n in zip(lengths_before, n_new) for p in range(a, a + n)]),
        tok_seq=i32([i for i, n in enumerate(n_new) for _ in range(n)]), cu_q=i32(cu), kv_len=i32(new_len),
        slots_dev=i32(slots), max_q_len=max(n_new),
        page_tables=[cache.page_table(g, slots).to(DEV) for g in range(len(cache.kv_groups))],
        cache_rows=[i32(cache.write_rows(g, slots, lengths_before, new_len).tolist())
                    for g in range(len(cache.kv_groups))], host_lengths=new_len)


def test_rmsnorm_part():
    n = RMSNorm(size=72, eps=1e-5, offset=1.0)
    w = torch.randn(72) * 0.1
    n.bind({"weight": w.to(DEV)})
    x = torch.randn(5, 72) * 4
    assert rel(n.apply(x.to(DEV), torch.float32), plain.rms_norm(x, w, 1e-5)) <= 2e-6
    n0 = RMSNorm(size=72, eps=1e-5, offset=0.0)
    n0.bind({"weight": (1 + w).to(DEV)})
    assert rel(n0.apply(x.to(DEV), torch.float32), plain.rms_norm(x, w, 1e-5)) <= 2e-6


def test_rotary_table():
    r = RotaryEmbedding(head_dim=48, theta=777.0)
    r.prepare(300, DEV)
    i = torch.arange(24, dtype=torch.float64)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * (777.0 ** (-2 * i / 48))[None]
    assert float((r.table[..., 0].double().cpu() - ang.cos()).abs().max()) < 1e-7
    assert float((r.table[..., 1].double().cpu() - ang.sin()).abs().max()) < 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_prompt_then_decode(dtype, window):
    hidden, n_q, n_kv, hd, theta, scale, cap = 80, 6, 2, 32, 500.0, 0.21, 25.0
    rope = RotaryEmbedding(hd, theta)
    att = Attention(hidden, n_q, n_kv, hd, scale, cap, window, rope)
    g = torch.Generator().manual_seed(1)
    ws = {n: (torch.randn(s.shape, generator=g) * 0.08).to(dtype) for n, s in att.param_specs().items()}
    att.bind({n: t.to(DEV) for n, t in ws.items()})
    cache = Cache([att.cache_spec()], 512, dtype, DEV)
    att.prepare(512, DEV)
    lengths = [90, 3]
    xs = [(torch.randn(n + 2, hidden, generator=g)).to(dtype) for n in lengths]

    def oracle(x):
        pos = torch.arange(x.shape[0])
        q = plain.rope(plain.linear(x, ws["q"]), pos, hd, theta)
        k = plain.rope(plain.linear(x, ws["k"]), pos, hd, theta)
        a = plain.attention(q, k, plain.linear(x, ws["v"]), n_q, n_kv, hd, scale, cap, window or 0)
        return plain.linear(a, ws["o"])

    refs = [oracle(x) for x in xs]
    ctx = make_ctx(cache, "prefill", [0, 0], lengths, dtype)
    y = att.forward(torch.cat([x[:n] for x, n in zip(xs, lengths)]).to(DEV), ctx, cache.entries[0])
    assert y.dtype == torch.float32
    if y.dim() == 3:            # partial sums along K, which the residual kernel would add
        y = y.sum(0)
    assert rel(y[:90], refs[0][:90]) <= TOL[dtype] and rel(y[90:], refs[1][:3]) <= TOL[dtype]
    for step in range(2):
        ctx = make_ctx(cache, "decode", [n + step for n in lengths], [1, 1], dtype)
        y = att.forward(torch.stack([x[n + step] for x, n in zip(xs, lengths)]).to(DEV), ctx, cache.entries[0])
        y = y.sum(0) if y.dim() == 3 else y
        for b in range(2):
            assert rel(y[b], refs[b][lengths[b] + step]) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    ffn = GatedFeedForward(hidden=72, inter=200, activation="gelu_tanh")
    g = torch.Generator().manual_seed(2)
    ws = {n: (torch.randn(s.shape, generator=g) * 0.1).to(dtype) for n, s in ffn.param_specs().items()}
    ffn.bind({n: t.to(DEV) for n, t in ws.items()})
    x = torch.randn(9, 72, generator=g).to(dtype)

    class Ctx:
        pass
    ctx = Ctx()
    ctx.dtype = dtype
    y = ffn.forward(x.to(DEV), ctx)
    y = y.sum(0) if y.dim() == 3 else y
    assert rel(y, plain.feed_forward(x, ws["gate"], ws["up"], ws["down"])) <= TOL[dtype]


def test_block_without_post_norms():
    """The pre-norm arrangement: h += mixer(pre(h)); h += ffn(pre(h))."""
    hidden, dtype = 64, torch.float32
    g = torch.Generator().manual_seed(3)

    def norm():
        n = RMSNorm(hidden, 1e-6, 0.0)
        n.w = torch.randn(hidden, generator=g) * 0.1 + 1
        n.bind({"weight": n.w.to(DEV)})
        return n

    att = Attention(hidden, 2, 2, 32, 32 ** -0.5, 0.0, None, None)     # no position encoding at all
    ffn = GatedFeedForward(hidden, 96, "silu")
    wa = {n: torch.randn(s.shape, generator=g) * 0.1 for n, s in att.param_specs().items()}
    wf = {n: torch.randn(s.shape, generator=g) * 0.1 for n, s in ffn.param_specs().items()}
    att.bind({n: t.to(DEV) for n, t in wa.items()})
    ffn.bind({n: t.to(DEV) for n, t in wf.items()})
    n1, n2, n3 = norm(), norm(), norm()
    blk = Block(att, ffn, n1, n2)
    cache = Cache([att.cache_spec()], 128, dtype, DEV)
    ctx = make_ctx(cache, "prefill", [0], [10], dtype)
    h0 = torch.randn(10, hidden, generator=g)
    h = h0.clone().to(DEV)
    x_next = blk.forward(h, n1.apply(h, dtype), ctx, cache.entries[0], True, n3)

    def pn(x, n):
        return plain.rms_norm(x, n.w - 1, 1e-6)
    x = pn(h0, n1)
    a = plain.attention(plain.linear(x, wa["q"]), plain.linear(x, wa["k"]), plain.linear(x, wa["v"]), 2, 2, 32,
                        32 ** -0.5, 0.0, 0)
    h1 = h0.double() + plain.linear(a, wa["o"])
    x = pn(h1, n2)
    gate = plain.linear(x, wf["gate"])
    h2 = h1 + plain.linear(gate * torch.sigmoid(gate) * plain.linear(x, wf["up"]), wf["down"])
    assert rel(h, h2) <= 2e-5
    assert rel(x_next, pn(h2, n3)) <= 2e-5
