"""The decode chain kernel alone: each kind of operation against plain float64
PyTorch, at sizes that are not the engine's, then operations in a row (the
barrier between them), launched twice (the barrier's words reset themselves)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _mods():
    from brolm_b200 import kernels
    from brolm_b200.engine import fused
    from brolm_b200.parts.norm import RMSNorm
    return kernels, fused, RMSNorm


def _norm(RMSNorm, size, eps, offset, gen):
    n = RMSNorm(size, eps, offset)
    n.bind({"weight": (torch.randn(size, generator=gen) * 0.3).to(DEV).bfloat16()})
    return n


def _x(rows_live, K, gen, fused):
    x = torch.zeros(fused.ROWS, K, dtype=torch.bfloat16, device=DEV)
    x[:rows_live] = torch.randn(rows_live, K, generator=gen).to(DEV).bfloat16()
    return x


def _run(kernels, b, M, positions=None, cache_rows=(), times=1):
    maps, ops, sync = b.finish()
    pos = positions if positions is not None else torch.zeros(16, dtype=torch.int32, device=DEV)
    for _ in range(times):
        kernels.decode_chain(maps, ops, 0, len(b), M, pos, list(cache_rows), sync)
    torch.cuda.synchronize()
    assert kernels.decode_chain_status(reset=True) == 0
    assert sync.tolist() == [0, 0, 0, 0]


def _rms(v, w, eps, offset):
    return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * (offset + w.double())


@pytest.mark.parametrize("N,K,M,max_split", [(200, 72, 3, 8), (2304, 2048, 8, 8), (4096, 2304, 16, 8), (136, 640, 1, 1),
                                             (520, 4104, 7, 5)])
def test_product_partial_sums(N, K, M, max_split):
    kernels, fused, _ = _mods()
    g = torch.Generator().manual_seed(N + K)
    w = (torch.randn(N, K, generator=g) * 0.05).to(DEV).bfloat16()
    x = _x(M, K, g, fused)
    b = fused.ChainBuilder(DEV)
    parts = b.gemm(w, x, "y", kernels.CHAIN_PARTS, max_split=max_split)
    parts.fill_(float("nan"))
    _run(kernels, b, M)
    want = x[:M].double() @ w.double().t()
    got = parts[:, :M].double().sum(0)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item())
    assert torch.isnan(parts[:, M:]).all()                     # rows that are not live are not written


@pytest.mark.parametrize("inter,K,M,act", [(328, 96, 5, "gelu_tanh"), (9216, 2304, 8, "gelu_tanh"), (64, 64, 16, "silu")])
def test_gated_product(inter, K, M, act):
    kernels, fused, _ = _mods()
    g = torch.Generator().manual_seed(inter)
    w = (torch.randn(2 * inter, K, generator=g) * 0.08).to(DEV).bfloat16()
    x = _x(M, K, g, fused)
    b = fused.ChainBuilder(DEV)
    out = torch.zeros(fused.ROWS, inter, dtype=torch.bfloat16, device=DEV)
    b.gemm(w, x, out, kernels.CHAIN_GATED, activation=act)
    _run(kernels, b, M)
    y = x[:M].double() @ w.double().t()
    gate, up = y[:, :inter], y[:, inter:]
    if act == "silu":
        a = gate * torch.sigmoid(gate)
    else:
        a = 0.5 * gate * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (gate + 0.044715 * gate ** 3)))
    want = a * up
    err = (out[:M].double() - want).abs()
    assert (err <= 2.0 ** -8 * want.abs() + 1e-6 * want.abs().max()).all()      # one bfloat16 rounding
    assert (out[M:] == 0).all()


def test_soft_capped_product():
    kernels, fused, _ = _mods()
    g = torch.Generator().manual_seed(5)
    N, K, M, cap = 500, 96, 6, 15.0
    w = (torch.randn(N, K, generator=g) * 0.6).to(DEV).bfloat16()
    x = _x(M, K, g, fused)
    b = fused.ChainBuilder(DEV)
    out = torch.zeros(fused.ROWS, N, dtype=torch.float32, device=DEV)
    b.gemm(w, x, out, kernels.CHAIN_SOFTCAP, cap=cap)
    _run(kernels, b, M)
    want = cap * torch.tanh(x[:M].double() @ w.double().t() / cap)
    assert want.abs().max() > 0.9 * cap                         # the cap does something here
    assert (out[:M].double() - want).abs().max().item() <= 2e-5 * cap


@pytest.mark.parametrize("H,inter,M", [(96, 328, 5), (2304, 1024, 8), (4608, 256, 2)])
def test_operations_in_a_row(H, inter, M):
    """norm -> gated product -> product in K slices -> norm: every operation reads what the one
    before it wrote, through the barrier; twice with the same barrier words."""
    kernels, fused, RMSNorm = _mods()
    g = torch.Generator().manual_seed(H)
    post0, pre, post1, nxt = (_norm(RMSNorm, H, e, o, g) for e, o in ((1e-6, 1.0), (1e-5, 1.0), (1e-6, 0.0), (1e-5, 1.0)))
    w_gu = (torch.randn(2 * inter, H, generator=g) * 0.05).to(DEV).bfloat16()
    w_d = (torch.randn(H, inter, generator=g) * 0.05).to(DEV).bfloat16()
    b = fused.ChainBuilder(DEV)
    h = b.buffer("h", (fused.ROWS, H), torch.float32)
    h0 = torch.randn(M, H, generator=g).to(DEV)
    y0 = torch.zeros(3, fused.ROWS, H, device=DEV)
    y0[:, :M] = torch.randn(3, M, H, generator=g).to(DEV)
    x = b.buffer("x", (fused.ROWS, H), torch.bfloat16)
    act = b.buffer("act", (fused.ROWS, inter), torch.bfloat16)
    b.norm(h, y0, post0, pre, x)
    b.gemm(w_gu, x, act, kernels.CHAIN_GATED)
    d = b.gemm(w_d, act, "d", kernels.CHAIN_PARTS)
    x2 = b.buffer("x2", (fused.ROWS, H), torch.bfloat16)
    b.norm(h, d, post1, nxt, x2)
    outs = []
    for _ in range(2):
        h[:M] = h0
        _run(kernels, b, M)
        outs.append((h[:M].clone(), x2[:M].clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])

    h1 = h0.double() + _rms(y0[:, :M].double().sum(0), post0.weight, post0.eps, post0.offset)
    xa = _rms(h1, pre.weight, pre.eps, pre.offset).to(torch.bfloat16).double()
    gu = xa @ w_gu.double().t()
    gate, up = gu[:, :inter], gu[:, inter:]
    a = (0.5 * gate * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (gate + 0.044715 * gate ** 3))) * up)
    a = a.to(torch.bfloat16).double()
    h2 = h1 + _rms(a @ w_d.double().t(), post1.weight, post1.eps, post1.offset)
    x_want = _rms(h2, nxt.weight, nxt.eps, nxt.offset)
    # the reference rounds the activations to bfloat16 where the kernel does; the residual stream is float
    assert (outs[0][0].double() - h2).abs().max().item() <= 2e-3 * h2.abs().max().item()
    assert (outs[0][1].double() - x_want).abs().max().item() <= 1e-2 * x_want.abs().max().item()


@pytest.mark.parametrize("n_q,n_kv,hd,rot,M", [(4, 2, 16, 16, 5), (8, 4, 256, 256, 8), (6, 1, 32, 16, 3)])
def test_rotation_and_cache_write(n_q, n_kv, hd, rot, M):
    kernels, fused, _ = _mods()
    g = torch.Generator().manual_seed(hd + n_q)
    width, page, pages = (n_q + 2 * n_kv) * hd, 64, 5
    parts = torch.zeros(2, fused.ROWS, width, device=DEV)
    parts[:, :M] = torch.randn(2, M, width, generator=g).to(DEV)
    out = torch.full((fused.ROWS, width), 7.0, dtype=torch.bfloat16, device=DEV)
    k_pages = torch.zeros(pages, n_kv, page, hd, dtype=torch.bfloat16, device=DEV)
    v_pages = torch.zeros_like(k_pages)
    half = rot // 2
    pos = torch.tensor([3, 70, -1, 0, 129, 5, 6, 7][:M] + [0] * (16 - M), dtype=torch.int32, device=DEV)
    crow = torch.tensor([3, 64 + 6, 9, -1, 2 * 64 + 1, 200, 201, 202][:M] + [-1] * (16 - M), dtype=torch.int32,
                        device=DEV)
    ang = torch.arange(256, dtype=torch.float64)[:, None] * (10000.0 ** (-2.0 * torch.arange(half, dtype=torch.float64) / rot))
    table = torch.stack([ang.cos(), ang.sin()], -1).float().to(DEV).contiguous()
    b = fused.ChainBuilder(DEV)
    b.rope(parts, out, table, rot, n_q, n_kv, hd, k_pages, v_pages, page, group=1)
    dummy = torch.zeros(16, dtype=torch.int32, device=DEV)
    _run(kernels, b, M, positions=pos, cache_rows=[dummy, crow])

    src = parts[:, :M].double().sum(0).view(M, n_q + 2 * n_kv, hd)
    want = src.clone()
    for t in range(M):
        p = int(pos[t])
        if p < 0:
            continue
        c, s = table[p, :, 0].double(), table[p, :, 1].double()
        a, bb = src[t, :n_q + n_kv, :half], src[t, :n_q + n_kv, half:rot]
        want[t, :n_q + n_kv, :half] = a * c - bb * s
        want[t, :n_q + n_kv, half:rot] = a * s + bb * c
    got = out[:M].double().view(M, n_q + 2 * n_kv, hd)
    for t in range(M):
        if int(pos[t]) < 0:
            assert (got[t] == 7.0).all()                        # a padding row is left alone
            continue
        assert (got[t] - want[t]).abs().max().item() <= 2.0 ** -8 * want[t].abs().max().item()
        r = int(crow[t])
        if r >= 0:
            kk, vv = k_pages[r // page, :, r % page].double(), v_pages[r // page, :, r % page].double()
            assert torch.equal(kk, got[t, n_q:n_q + n_kv]) and torch.equal(vv, got[t, n_q + n_kv:])
    kept = {int(r) for t, r in enumerate(crow[:M].tolist()) if r >= 0 and int(pos[t]) >= 0}
    mask = torch.ones(pages * page, dtype=torch.bool)
    mask[list(kept)] = False
    assert (k_pages.permute(0, 2, 1, 3).reshape(pages * page, -1)[mask.to(DEV)] == 0).all()   # nothing else written


def test_refuses_more_rows_than_it_takes():
    kernels, fused, _ = _mods()
    b = fused.ChainBuilder(DEV)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    b.gemm(w, torch.zeros(fused.ROWS, 64, dtype=torch.bfloat16, device=DEV), "y", kernels.CHAIN_PARTS)
    maps, ops, sync = b.finish()
    with pytest.raises(kernels.KernelError):
        kernels.decode_chain(maps, ops, 0, 1, 17, torch.zeros(32, dtype=torch.int32, device=DEV), [], sync)


@pytest.mark.parametrize("graphs", [False, True])
def test_engine_decodes_through_chains(tmp_path, monkeypatch, graphs):
    """With BROLM_CHAIN=1 the engine's decode steps run as chains: unequal batches, one after another on
    the same slots, token by token against the plain implementation; and whole versus one by one."""
    import brolm_b200 as bb
    from tests.helpers import make_folder, oracle_inputs, random_prompts
    from tests.plain import gemma2_plain as plain
    from tests.test_engine_gpu import check, run_batch_teacher_forced
    monkeypatch.setenv("BROLM_CHAIN", "1")
    for name in ("A", "B"):
        folder = make_folder(tmp_path, name, torch.bfloat16)
        config, weights = oracle_inputs(folder)
        model = bb.load_model(folder, dtype="bfloat16", device=DEV)
        eng = bb.Engine(model, max_tokens=64 * 8, max_slots=4, use_graphs=graphs)
        V = config["vocab_size"]
        run_batch_teacher_forced(eng, config, weights, random_prompts(V, [9, 100, 40, 150], 21), [5, 90, 1, 140],
                                 "bfloat16")
        run_batch_teacher_forced(eng, config, weights, random_prompts(V, [70, 3, 33], 22), [60, 1, 20], "bfloat16")
        assert model._chain_why == "" and len(model._chain_plans) == 1          # the chains did run
        p = random_prompts(V, [90], 23)[0]
        ref = plain.forward(config, weights, p)
        (s,) = eng.open(1)
        eng.step([s], [p[:50]])
        for i in range(50, len(p)):
            check(eng.step([s], [[p[i]]])[0], ref[i], "bfloat16", f"token {i} decoded alone through a chain")
        eng.close([s])
