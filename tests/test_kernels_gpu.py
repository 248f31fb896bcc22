"""Each kernel alone against a plain float64 torch restatement, at sizes
other than the engine's (widths and vocabularies that are no power of two,
head sizes in steps of 16, odd head counts)."""
import math

import pytest
import torch

from brolm_b200 import kernels
from tests.plain import gemma2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 2e-6, torch.bfloat16: 8e-3}   # relative to the largest magnitude of the result


def close(got, ref, dtype, scale=None):
    ref = ref.double().cpu()
    got = got.double().cpu()
    s = scale if scale is not None else max(1e-30, float(ref.abs().max()))
    err = float((got - ref).abs().max()) / s
    assert err <= TOL[dtype], f"error {err:.3e} exceeds {TOL[dtype]:.1e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_scale(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1000, 200, generator=g).to(dtype)
    ids = torch.randint(0, 1000, (37,), generator=g, dtype=torch.int32)
    out = torch.empty(37, 200, dtype=torch.float32, device=DEV)
    kernels.embed_scale(ids.to(DEV), table.to(DEV), math.sqrt(200.0), out)
    ref = plain.embed(table, ids, 200)
    close(out, ref, torch.float32)


@pytest.mark.parametrize("xd,wd,od", [(torch.float32, torch.float32, torch.float32),
                                       (torch.float32, torch.bfloat16, torch.bfloat16),
                                       (torch.bfloat16, torch.float32, torch.bfloat16),
                                       (torch.float32, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("hidden", [200, 2304])
def test_rmsnorm(xd, wd, od, hidden):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(19, hidden, generator=g) * 3).to(xd)
    w = (torch.randn(hidden, generator=g) * 0.1).to(wd)
    out = torch.empty(19, hidden, dtype=od, device=DEV)
    kernels.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, 1.0, out)
    close(out, plain.rms_norm(x, w, 1e-5), od)
    rows = torch.tensor([18, 0, 7], dtype=torch.int32)
    out2 = torch.empty(3, hidden, dtype=od, device=DEV)
    kernels.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, 1.0, out2, rows.to(DEV))
    close(out2, plain.rms_norm(x[rows.long()], w, 1e-5), od)


@pytest.mark.parametrize("yd,wd,od", [(torch.float32, torch.float32, torch.float32),
                                       (torch.float32, torch.bfloat16, torch.bfloat16),
                                       (torch.bfloat16, torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("post,nxt", [(True, True), (True, False), (False, True), (False, False)])
def test_residual_rmsnorm(yd, wd, od, post, nxt):
    hidden = 328
    g = torch.Generator().manual_seed(2)
    h = torch.randn(11, hidden, generator=g) * 5
    y = (torch.randn(11, hidden, generator=g) * 2).to(yd)
    w1 = (torch.randn(hidden, generator=g) * 0.1).to(wd)
    w2 = (torch.randn(hidden, generator=g) * 0.1).to(wd)
    hd = h.clone().to(DEV)
    out = torch.empty(11, hidden, dtype=od, device=DEV) if nxt else None
    kernels.residual_rmsnorm(hd, y.to(DEV), w1.to(DEV) if post else None, 1e-6, 1.0,
                             w2.to(DEV) if nxt else None, 1e-5, 1.0, out)
    h_ref = h.double() + (plain.rms_norm(y, w1, 1e-6) if post else y.double())
    close(hd, h_ref, torch.float32)
    if nxt:
        close(out, plain.rms_norm(h_ref, w2, 1e-5), od)


@pytest.mark.parametrize("rows,hidden", [(1500, 2304), (2000, 328), (1300, 3584), (1185, 1024), (5000, 2304)])
@pytest.mark.parametrize("post,nxt", [(True, True), (False, True), (True, False)])
def test_residual_rmsnorm_of_a_prompts_rows(rows, hidden, post, nxt):
    """Thousands of rows (a prompt): the form with the row in shared memory, at one and at several rounds of
    its blocks and at widths of one to four chunks per thread."""
    g = torch.Generator().manual_seed(rows + hidden)
    h = torch.randn(rows, hidden, generator=g) * 5
    y = (torch.randn(rows, hidden, generator=g) * 2).to(torch.bfloat16)
    w1 = (torch.randn(hidden, generator=g) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn(hidden, generator=g) * 0.1).to(torch.bfloat16)
    hd = h.clone().to(DEV)
    out = torch.full((rows, hidden), float("nan"), dtype=torch.bfloat16, device=DEV) if nxt else None
    kernels.residual_rmsnorm(hd, y.to(DEV), w1.to(DEV) if post else None, 1e-6, 1.0,
                             w2.to(DEV) if nxt else None, 1e-5, 1.0, out)
    h_ref = h.double() + (plain.rms_norm(y, w1, 1e-6) if post else y.double())
    close(hd, h_ref, torch.float32)
    if nxt:
        close(out, plain.rms_norm(h_ref, w2, 1e-5), torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_gated_act(dtype, act):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(7, 2 * 330, generator=g) * 3).to(dtype)
    out = torch.empty(7, 330, dtype=dtype, device=DEV)
    kernels.gated_act(gu.to(DEV), out, act)
    gate, up = gu[:, :330].double(), gu[:, 330:].double()
    ref = (plain.gelu_tanh(gate) if act == "gelu_tanh" else gate * torch.sigmoid(gate)) * up
    close(out, ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softcap(dtype):
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(3, 1001, generator=g) * 40).to(dtype)
    out = torch.empty(3, 1001, dtype=torch.float32, device=DEV)
    kernels.softcap(x.to(DEV), out, 30.0)
    close(out, plain.soft_cap(x.double(), 30.0), torch.float32)
    assert float(out.abs().max()) <= 30.0
    kernels.softcap(x.to(DEV), out, 0.0)
    close(out, x.double(), torch.float32)


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 96), (65, 200, 330), (128, 64, 16), (17, 1000, 203)])
def test_linear_f32(M, N, K):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    kernels.linear_f32(x.to(DEV), w.to(DEV), out)
    close(out, plain.linear(x, w), torch.float32)
    # a row gives the same bits alone and in the batch
    one = torch.empty(1, N, dtype=torch.float32, device=DEV)
    kernels.linear_f32(x[M - 1:M].to(DEV), w.to(DEV), one)
    assert torch.equal(one[0], out[M - 1])


def test_linear_f32_strided_views():
    g = torch.Generator().manual_seed(6)
    big = torch.randn(9, 3 * 48, generator=g).to(DEV)
    w = torch.randn(20, 48, generator=g).to(DEV)
    out = torch.zeros(9, 64, dtype=torch.float32, device=DEV)
    kernels.linear_f32(big[:, 48:96], w, out[:, 8:28])
    close(out[:, 8:28], plain.linear(big[:, 48:96].cpu(), w.cpu()), torch.float32)
    assert float(out[:, :8].abs().max()) == 0 and float(out[:, 28:].abs().max()) == 0


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(16, 64), (40, 72), (1000, 200), (2304, 2304), (48, 9216)])
def test_skinny_gemm(M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    ref = plain.linear(x, w)
    for dt in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), 7.0, dtype=dt, device=DEV)
        kernels.skinny_gemm(x.to(DEV), w.to(DEV), out)
        close(out, ref, torch.float32 if dt == torch.float32 else torch.bfloat16,
              scale=float(ref.abs().max()) * (50 if dt == torch.float32 else 1))
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    kernels.skinny_gemm(x.to(DEV), w.to(DEV), out, "softcap", cap=3.0)
    close(out, plain.soft_cap(ref, 3.0), torch.float32, scale=3.0 * 50)
    # a row gives the same bits alone and in the batch
    one = torch.empty(1, N, dtype=torch.float32, device=DEV)
    kernels.skinny_gemm(x[M - 1:M].to(DEV), w.to(DEV), one, "softcap", cap=3.0)
    assert torch.equal(one[0], out[M - 1])


@pytest.mark.parametrize("M,F,K,act", [(1, 16, 64, "gelu_tanh"), (8, 328, 96, "silu"), (13, 9216, 128, "gelu_tanh"),
                                       (16, 40, 2304, "gelu_tanh")])
def test_skinny_gemm_gated(M, F, K, act):
    g = torch.Generator().manual_seed(F + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, generator=g) * 0.1).to(torch.bfloat16)
    gate, up = plain.linear(x, w[:F]), plain.linear(x, w[F:])
    ref = (plain.gelu_tanh(gate) if act == "gelu_tanh" else gate * torch.sigmoid(gate)) * up
    out = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
    kernels.skinny_gemm(x.to(DEV), w.to(DEV), out, "gated", act)
    close(out, ref, torch.bfloat16)


@pytest.mark.parametrize("parts", [2, 3, 8])
def test_skinny_gemm_partial_sums_feed_the_residual_kernel(parts):
    g = torch.Generator().manual_seed(parts)
    M, N, K = 5, 328, 9216
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    y = torch.full((parts, M, N), float("nan"), dtype=torch.float32, device=DEV)
    kernels.skinny_gemm(x.to(DEV), w.to(DEV), y)
    ref = plain.linear(x, w)
    close(y.sum(0), ref, torch.float32, scale=float(ref.abs().max()) * 50)
    h = torch.randn(M, N, generator=g)
    gain = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16)
    hd_ = h.clone().to(DEV)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.residual_rmsnorm(hd_, y, gain.to(DEV), 1e-6, 1.0, gain.to(DEV), 1e-6, 1.0, out)
    h_ref = h.double() + plain.rms_norm(ref, gain, 1e-6)
    close(hd_, h_ref, torch.float32, scale=float(h_ref.abs().max()) * 50)
    close(out, plain.rms_norm(h_ref, gain, 1e-6), torch.bfloat16)
    assert kernels.skinny_parts(torch.empty(8, 9216), torch.empty(2304, 9216), sms=148) == 3
    assert kernels.skinny_parts(torch.empty(8, 2304), torch.empty(18432, 2304)) == 1


@pytest.mark.parametrize("pairs", [True, False])
@pytest.mark.parametrize("M,N,K", [(17, 256, 64), (128, 256, 256), (100, 300, 200), (333, 2304, 2048), (1000, 40, 72),
                                   (2048, 512, 9216), (257, 520, 136)])
def test_gemm_tc(M, N, K, pairs):
    """One block per 128 x 256 tile, and a pair of SMs per 256 x 256 tile (cta_group::2)."""
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    ref = plain.linear(x, w)
    for dt in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), 7.0, dtype=dt, device=DEV)
        kernels.gemm_tc(x.to(DEV), w.to(DEV), out, pairs=pairs)
        close(out, ref, dt, scale=float(ref.abs().max()) * (50 if dt == torch.float32 else 1))
    assert kernels.gemm_tc_status() == 0


@pytest.mark.parametrize("pairs", [True, False])
@pytest.mark.parametrize("M,F,K,act", [(17, 128, 64, "gelu_tanh"), (300, 384, 200, "silu"), (2048, 9216, 2304, "gelu_tanh")])
def test_gemm_tc_gated(M, F, K, act, pairs):
    g = torch.Generator().manual_seed(F + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, generator=g) * 0.05).to(torch.bfloat16)
    xd, wd = x.to(DEV), w.to(DEV)
    out = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_tc(xd, wd, out, "gated", act, pairs=pairs)
    gate, up = xd.double() @ wd[:F].double().t(), xd.double() @ wd[F:].double().t()      # float64 on the device: fast
    ref = (plain.gelu_tanh(gate) if act == "gelu_tanh" else gate * torch.sigmoid(gate)) * up
    close(out, ref, torch.bfloat16)
    assert kernels.gemm_tc_status() == 0


@pytest.mark.parametrize("M,N,K,parts", [(1, 128, 256, 1), (8, 2304, 2048, 8), (16, 300, 200, 1), (17, 4096, 2304, 1),
                                         (64, 2304, 9216, 8), (128, 512, 512, 3), (33, 1000, 72, 1)])
def test_gemm_stream(M, N, K, parts):
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ref = x.double() @ w.double().t()
    for dt in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), 7.0, dtype=dt, device=DEV)
        kernels.gemm_stream(x, w, out)
        close(out, ref, dt, scale=float(ref.abs().max()) * (50 if dt == torch.float32 else 1))
    if parts > 1:
        nkb = (K + 63) // 64
        per = (nkb + parts - 1) // parts
        parts = (nkb + per - 1) // per                      # no empty slice
        y = torch.full((parts, M, N), float("nan"), dtype=torch.float32, device=DEV)
        kernels.gemm_stream(x, w, y)
        close(y.sum(0), ref, torch.float32, scale=float(ref.abs().max()) * 50)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    kernels.gemm_stream(x, w, out, "softcap", cap=3.0)
    close(out, plain.soft_cap(ref, 3.0), torch.float32, scale=3.0 * 50)
    assert kernels.gemm_stream_status() == 0


@pytest.mark.parametrize("M,F,K,act", [(1, 64, 64, "gelu_tanh"), (8, 9216, 2304, "gelu_tanh"), (50, 128, 72, "silu"),
                                       (100, 320, 128, "gelu_tanh")])
def test_gemm_stream_gated(M, F, K, act):
    g = torch.Generator().manual_seed(F + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * F, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    out = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_stream(x, w, out, "gated", act)
    gate, up = x.double() @ w[:F].double().t(), x.double() @ w[F:].double().t()
    ref = (plain.gelu_tanh(gate) if act == "gelu_tanh" else gate * torch.sigmoid(gate)) * up
    close(out, ref, torch.bfloat16)
    assert kernels.gemm_stream_status() == 0
    # o of Gemma 2 2B (32 blocks of K, 18 row tiles): a ring's worth of K per item, four slices
    assert kernels.gemm_stream_parts(torch.empty(8, 2048), torch.empty(2304, 2048)) == 4
    assert kernels.gemm_stream_parts(torch.empty(8, 9216), torch.empty(2304, 9216)) == 8
    assert kernels.gemm_stream_parts(torch.empty(8, 2304), torch.empty(256000, 2304)) == 1


def test_gemm_tc_strided_views():
    g = torch.Generator().manual_seed(2)
    big = torch.randn(40, 3 * 64, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(24, 64, generator=g).to(torch.bfloat16).to(DEV)
    x = big[:, 64:128]
    assert kernels.gemm_tc_ok(x, w, sms=1) and not kernels.gemm_tc_ok(big[:, 1:65], w, sms=1)
    assert not kernels.gemm_tc_ok(x, w)            # one tile only: not worth a persistent kernel
    wide = torch.zeros(40, 64, dtype=torch.float32, device=DEV)
    kernels.gemm_tc(x, w, wide[:, 8:32])
    close(wide[:, 8:32], plain.linear(x.cpu(), w.cpu()), torch.float32, scale=float(wide.abs().max()) * 50)
    assert float(wide[:, :8].abs().max()) == 0 and float(wide[:, 32:].abs().max()) == 0


def test_skinny_gemm_strided_input():
    g = torch.Generator().manual_seed(1)
    big = torch.randn(5, 3 * 64, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(24, 64, generator=g).to(torch.bfloat16).to(DEV)
    x = big[:, 64:128]
    assert kernels.skinny_ok(x, w) and not kernels.skinny_ok(big[:, 1:65], w)
    out = torch.empty(5, 24, dtype=torch.float32, device=DEV)
    kernels.skinny_gemm(x, w, out)
    close(out, plain.linear(x.cpu(), w.cpu()), torch.float32, scale=float(out.abs().max()) * 50)


def _rope_case(dtype, n_q, n_kv, hd, ring, page, lengths, seed):
    """Prompt pass of unequal sequences: rotation against the oracle and the pages written."""
    g = torch.Generator().manual_seed(seed)
    B = len(lengths)
    T = sum(lengths)
    width = (n_q + 2 * n_kv) * hd
    qkv = torch.randn(T, width, generator=g).to(dtype)
    positions = torch.cat([torch.arange(n) for n in lengths]).int()
    theta = 1000.0
    half = hd // 2
    inv = torch.tensor(theta, dtype=torch.float64) ** (-2.0 * torch.arange(half, dtype=torch.float64) / hd)
    ang = torch.arange(max(lengths), dtype=torch.float64)[:, None] * inv[None]
    table = torch.stack([ang.cos(), ang.sin()], -1).float()
    pages_per = [min((n + page - 1) // page, ring // page) for n in lengths]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()        # scattered page ids
    pt = torch.zeros(B, max(pages_per), dtype=torch.int32)
    it = iter(perm)
    for b in range(B):
        for j in range(pages_per[b]):
            pt[b, j] = next(it)
    kp = torch.zeros(n_pages, n_kv, page, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    dq = qkv.clone().to(DEV)
    rows = []
    for b, n in enumerate(lengths):
        for p_ in range(n):
            ridx = p_ % ring
            rows.append(int(pt[b, ridx // page]) * page + ridx % page if p_ >= n - ring else -1)
    kernels.rope_kv_write(dq, positions.to(DEV), table.to(DEV), n_q, n_kv, hd, hd, kp, vp,
                          torch.tensor(rows, dtype=torch.int32, device=DEV), page)
    q_ref = plain.rope(qkv[:, :n_q * hd], positions, hd, theta)
    k_ref = plain.rope(qkv[:, n_q * hd:(n_q + n_kv) * hd], positions, hd, theta)
    close(dq[:, :n_q * hd], q_ref, dtype)
    close(dq[:, n_q * hd:(n_q + n_kv) * hd], k_ref, dtype)
    assert torch.equal(dq[:, (n_q + n_kv) * hd:].cpu(), qkv[:, (n_q + n_kv) * hd:])
    kp, vp, dq = kp.cpu(), vp.cpu(), dq.cpu()
    t = 0
    for b, n in enumerate(lengths):
        for p in range(n):
            if p >= n - ring:
                ridx = p % ring
                pg = int(pt[b, ridx // page])
                assert torch.equal(kp[pg, :, ridx % page, :].reshape(-1), dq[t, n_q * hd:(n_q + n_kv) * hd]), (b, p)
                assert torch.equal(vp[pg, :, ridx % page, :].reshape(-1), dq[t, (n_q + n_kv) * hd:]), (b, p)
            t += 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_kv_write_all_keys(dtype):
    _rope_case(dtype, n_q=6, n_kv=3, hd=48, ring=1 << 30, page=64, lengths=[1, 70, 130], seed=7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_kv_write_ring(dtype):
    # prompts longer than the ring: only the last `ring` places are written, each exactly once
    _rope_case(dtype, n_q=2, n_kv=1, hd=32, ring=64, page=32, lengths=[200, 64, 65, 3], seed=8)


@pytest.mark.parametrize("n_q,n_kv,hd,slices", [(8, 4, 256, 4), (6, 1, 32, 1), (3, 3, 48, 3), (32, 16, 128, 2)])
def test_rope_kv_write_from_partial_sums(n_q, n_kv, hd, slices):
    """The q/k/v projection as float slices of K: added in order, rotated, rounded once, written to the packed
    row and to the cache; a row with a negative position is left alone."""
    g = torch.Generator().manual_seed(hd + slices)
    T, page = 40, 64
    width = (n_q + 2 * n_kv) * hd
    parts = torch.randn(slices, T, width, generator=g)
    positions = torch.randint(0, 500, (T,), generator=g).int()
    positions[7] = -1
    theta = 1000.0
    inv = torch.tensor(theta, dtype=torch.float64) ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    ang = torch.arange(500, dtype=torch.float64)[:, None] * inv[None]
    table = torch.stack([ang.cos(), ang.sin()], -1).float()
    rows = torch.randperm(T * 2, generator=g)[:T].int()          # a place of its own for every token
    rows[11] = -1                                                 # a token the ring does not keep
    kp = torch.zeros(3, n_kv, page, hd, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    out = torch.full((T, width), 7.0, dtype=torch.bfloat16, device=DEV)
    kernels.rope_kv_write_parts(parts.to(DEV), out, positions.to(DEV), table.to(DEV), n_q, n_kv, hd, kp, vp,
                                rows.to(DEV), page)
    total = parts.double().sum(0)
    live = positions >= 0
    pos = positions.clamp(min=0)
    q_ref = plain.rope(total[:, :n_q * hd], pos, hd, theta)
    k_ref = plain.rope(total[:, n_q * hd:(n_q + n_kv) * hd], pos, hd, theta)
    ref = torch.cat([q_ref, k_ref, total[:, (n_q + n_kv) * hd:]], dim=1)
    close(out[live], ref[live], torch.bfloat16)
    assert float((out[7].float() - 7.0).abs().max()) == 0.0
    out, kp, vp = out.cpu(), kp.cpu(), vp.cpu()
    for t in range(T):
        if not live[t] or rows[t] < 0:
            continue
        pg, place = int(rows[t]) // page, int(rows[t]) % page
        assert torch.equal(kp[pg, :, place, :].reshape(-1), out[t, n_q * hd:(n_q + n_kv) * hd])
        assert torch.equal(vp[pg, :, place, :].reshape(-1), out[t, (n_q + n_kv) * hd:])
    written = (kp.float().abs().sum(-1) > 0).sum()
    assert int(written) == n_kv * int((live & (rows >= 0)).sum())   # nothing else was touched


def test_rope_skips_padding_rows():
    qkv = torch.randn(4, 4 * 16).to(DEV)
    before = qkv.clone()
    table = torch.zeros(8, 8, 2)
    table[..., 1] = 1.0   # a quarter turn everywhere
    pos = torch.tensor([-1, 2, -1, 3], dtype=torch.int32, device=DEV)
    kernels.rope_kv_write(qkv, pos, table.to(DEV), 2, 1, 16, 16)
    assert torch.equal(qkv[0], before[0]) and torch.equal(qkv[2], before[2])
    assert not torch.equal(qkv[1, :48], before[1, :48])


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def _attention_oracle(q, k, v, n_q, n_kv, hd, scale, cap, window):
    return plain.attention(q, k, v, n_q, n_kv, hd, scale, cap, window)


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "simt"), (torch.bfloat16, "simt"), (torch.bfloat16, "mma"),
                                          (torch.bfloat16, "tc")])
@pytest.mark.parametrize("n_q,n_kv,hd,window,cap", [(4, 2, 16, 8, 50.0), (6, 1, 32, 16, 20.0), (3, 3, 48, 0, 0.0),
                                                    (8, 4, 256, 100, 50.0), (5, 5, 128, 0, 30.0), (8, 1, 64, 33, 0.0),
                                                    (16, 1, 80, 70, 10.0), (4, 2, 64, 0, 50.0), (32, 16, 128, 0, 50.0),
                                                    (8, 8, 256, 0, 0.0)])
def test_attention_packed(dtype, kernel, n_q, n_kv, hd, window, cap):
    if kernel == "tc" and not kernels.attention_prefill_tc_ok(hd, n_q // n_kv):
        pytest.skip("sizes the tcgen05 kernel leaves to the mma.sync kernel")
    g = torch.Generator().manual_seed(hd + n_q)
    lengths = [1, 37, 150, 64, 300]
    T = sum(lengths)
    width = (n_q + 2 * n_kv) * hd
    qkv = (torch.randn(T, width, generator=g)).to(dtype)
    scale = 0.7 / math.sqrt(hd)
    dq = qkv.to(DEV)
    out = torch.empty(T, n_q * hd, dtype=dtype, device=DEV)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=DEV)
    kw = dict(n_kv=n_kv, group=n_q // n_kv, head_dim=hd, scale=scale, cap=cap, window=window,
              batch=len(lengths), max_q_len=max(lengths))
    kk, vv = dq[:, n_q * hd:(n_q + n_kv) * hd], dq[:, (n_q + n_kv) * hd:]
    if kernel == "mma":
        kernels.attention_prefill_mma(dq[:, :n_q * hd], out, cu, kk, vv, **kw)
    elif kernel == "tc":
        kernels.attention_prefill_tc(dq[:, :n_q * hd], out, cu, kk, vv, **kw)
        assert kernels.attention_tc_status() == 0
    else:
        kernels.attention_simt(dq[:, :n_q * hd], out, cu, torch.tensor(lengths, dtype=torch.int32, device=DEV),
                               k=kk, v=vv, **kw)
    t = 0
    for n in lengths:
        s = qkv[t:t + n]
        ref = _attention_oracle(s[:, :n_q * hd], s[:, n_q * hd:(n_q + n_kv) * hd], s[:, (n_q + n_kv) * hd:],
                                n_q, n_kv, hd, scale, cap, window)
        close(out[t:t + n], ref, dtype, scale=float(ref.abs().max()))
        t += n


@pytest.mark.parametrize("n_q,n_kv,hd,window,cap,gain", [(8, 4, 256, 0, 50.0, 40.0), (4, 2, 64, 100, 30.0, 25.0),
                                                         (4, 4, 128, 0, 20.0, 200.0)])
def test_attention_tc_scores_beyond_the_cap(n_q, n_kv, hd, window, cap, gain):
    """Queries scaled so that score * scale / cap runs from near 0 to far beyond 1, where tanh is flat and
    the row's reference maximum sits at the cap: tiles with small scores and tiles with saturated ones
    follow one another within a sequence."""
    g = torch.Generator().manual_seed(5)
    lengths = [300, 700, 129]
    T = sum(lengths)
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, generator=g)
    # rows 0-255 of each sequence keep small scores; later query rows are large
    t = 0
    for n in lengths:
        qkv[t + 256:t + n, :n_q * hd] *= gain
        t += n
    qkv = qkv.to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    dq = qkv.to(DEV)
    out = torch.empty(T, n_q * hd, dtype=torch.bfloat16, device=DEV)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=DEV)
    kernels.attention_prefill_tc(dq[:, :n_q * hd], out, cu, dq[:, n_q * hd:(n_q + n_kv) * hd], dq[:, (n_q + n_kv) * hd:],
                                 n_kv=n_kv, group=n_q // n_kv, head_dim=hd, scale=scale, cap=cap, window=window,
                                 batch=len(lengths), max_q_len=max(lengths))
    assert kernels.attention_tc_status() == 0
    t = 0
    for n in lengths:
        s = qkv[t:t + n]
        ref = _attention_oracle(s[:, :n_q * hd], s[:, n_q * hd:(n_q + n_kv) * hd], s[:, (n_q + n_kv) * hd:],
                                n_q, n_kv, hd, scale, cap, window)
        close(out[t:t + n], ref, torch.bfloat16, scale=float(ref.abs().max()))
        t += n


@pytest.mark.parametrize("n_q,n_kv,hd,window,cap,lengths", [(8, 4, 256, 512, 50.0, [1500, 130]),
                                                            (8, 4, 256, 0, 50.0, [2100]),
                                                            (4, 2, 128, 0, 30.0, [2100, 700])])
def test_attention_tc_long_prompts(n_q, n_kv, hd, window, cap, lengths):
    """Prompts of many key tiles: 1,500 tokens with a window of 512 (row blocks whose first key tile is
    not tile 0, windows that cut tiles at both ends) and 2,100 tokens without a window."""
    g = torch.Generator().manual_seed(11)
    T = sum(lengths)
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, generator=g).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    dq = qkv.to(DEV)
    out = torch.empty(T, n_q * hd, dtype=torch.bfloat16, device=DEV)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=DEV)
    kernels.attention_prefill_tc(dq[:, :n_q * hd], out, cu, dq[:, n_q * hd:(n_q + n_kv) * hd], dq[:, (n_q + n_kv) * hd:],
                                 n_kv=n_kv, group=n_q // n_kv, head_dim=hd, scale=scale, cap=cap, window=window,
                                 batch=len(lengths), max_q_len=max(lengths))
    assert kernels.attention_tc_status() == 0
    t = 0
    for n in lengths:
        s = qkv[t:t + n]
        ref = _attention_oracle(s[:, :n_q * hd], s[:, n_q * hd:(n_q + n_kv) * hd], s[:, (n_q + n_kv) * hd:],
                                n_q, n_kv, hd, scale, cap, window)
        close(out[t:t + n], ref, torch.bfloat16, scale=float(ref.abs().max()))
        t += n


@pytest.mark.parametrize("n_q,n_kv,hd,window,cap,lengths,n_split", [
    (8, 4, 256, 0, 50.0, [2048], None),            # the launcher's own choice (it cuts: 128 blocks on 148 SMs)
    (8, 4, 256, 0, 50.0, [1100], 9),               # every row block in two
    (8, 4, 256, 0, 50.0, [1100], 3),               # only the three heaviest
    (8, 4, 256, 300, 50.0, [1500], 24),            # a window: the first half of a row block ends before some rows' windows begin
    (4, 2, 128, 0, 30.0, [700, 64, 1, 130, 333], 6),   # sequences too short for the cut ranks, and ranks with one tile
    (4, 4, 64, 0, 0.0, [515, 900], 8),
    (2, 1, 256, 128, 50.0, [640], 5)])
def test_attention_tc_row_blocks_cut_in_two_along_the_keys(n_q, n_kv, hd, window, cap, lengths, n_split):
    """The heaviest row blocks as two halves of their keys, merged by the half that finishes second.  One far
    key per sequence (key 3, in the first half of every later row block) is made to carry almost all the
    weight of the last rows, so a lost or mis-scaled first half shows; twice over, so the tickets must have
    gone back to zero."""
    g = torch.Generator().manual_seed(17 + hd)
    T = sum(lengths)
    group = n_q // n_kv
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, generator=g)
    t = 0
    for n in lengths:
        if n > 200 and (window == 0 or window > n):
            key = qkv[t + 3, n_q * hd:n_q * hd + hd]
            qkv[t + n - 40:t + n, :hd] = key * 0.5           # head 0 of the last rows looks at key 3
        t += n
    qkv = qkv.to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    dq = qkv.to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=DEV)
    kw = dict(n_kv=n_kv, group=group, head_dim=hd, scale=scale, cap=cap, window=window, batch=len(lengths),
              max_q_len=max(lengths))
    if n_split is None:
        assert kernels.attention_prefill_tc_split(max(lengths), n_kv, group, window, len(lengths)) > 0
    whole = torch.empty(T, n_q * hd, dtype=torch.bfloat16, device=DEV)
    kernels.attention_prefill_tc(dq[:, :n_q * hd], whole, cu, dq[:, n_q * hd:(n_q + n_kv) * hd], dq[:, (n_q + n_kv) * hd:],
                                 n_split=0, **kw)
    for _ in range(2):
        out = torch.full((T, n_q * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        kernels.attention_prefill_tc(dq[:, :n_q * hd], out, cu, dq[:, n_q * hd:(n_q + n_kv) * hd], dq[:, (n_q + n_kv) * hd:],
                                     n_split=n_split, **kw)
        assert kernels.attention_tc_status() == 0
        t = 0
        for n in lengths:
            s_ = qkv[t:t + n]
            ref = _attention_oracle(s_[:, :n_q * hd], s_[:, n_q * hd:(n_q + n_kv) * hd], s_[:, (n_q + n_kv) * hd:],
                                    n_q, n_kv, hd, scale, cap, window)
            close(out[t:t + n], ref, torch.bfloat16, scale=float(ref.abs().max()))
            t += n
        # and close to the uncut kernel's result (the same products, another order of two sums)
        assert float((out.float() - whole.float()).abs().max()) <= 2e-2 * float(whole.float().abs().max())


def _paged_case(dtype, n_q, n_kv, hd, window, cap, lengths, page=64, special=None, seed=0, kernel="simt", splits=1):
    """Decode pass: one query per sequence over a scattered, possibly ring-shaped cache."""
    g = torch.Generator().manual_seed(seed)
    B = len(lengths)
    ring = ((window + page - 1) // page * page) if window else (1 << 30)
    scale = 1.0 / math.sqrt(hd)
    ks = [torch.randn(n, n_kv * hd, generator=g).to(dtype) for n in lengths]
    vs = [torch.randn(n, n_kv * hd, generator=g).to(dtype) for n in lengths]
    qs = [torch.randn(1, n_q * hd, generator=g).to(dtype) for _ in lengths]
    if special is not None:
        special(qs, ks, vs)
    pages_per = [min((n + page - 1) // page, ring // page) for n in lengths]
    n_pages = sum(pages_per) + 2
    perm = iter(torch.randperm(n_pages, generator=g).tolist())
    pt = torch.zeros(B, max(pages_per), dtype=torch.int32)
    kp = torch.full((n_pages, n_kv, page, hd), float("nan")).to(dtype)   # what is never written must never be read
    vp = kp.clone()
    for b, n in enumerate(lengths):
        for j in range(pages_per[b]):
            pt[b, j] = next(perm)
        for p in range(max(0, n - ring), n):
            ridx = p % ring
            kp[int(pt[b, ridx // page]), :, ridx % page, :] = ks[b][p].view(n_kv, hd)
            vp[int(pt[b, ridx // page]), :, ridx % page, :] = vs[b][p].view(n_kv, hd)
    q = torch.cat(qs).to(DEV)
    out = torch.empty(B, n_q * hd, dtype=dtype, device=DEV)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    kvl = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    kw = dict(n_kv=n_kv, group=n_q // n_kv, head_dim=hd, scale=scale, cap=cap, window=window, batch=B)
    if kernel == "mma":
        kernels.attention_decode_mma(q, out, cu, kvl, kp.to(DEV), vp.to(DEV), pt.to(DEV), ring=ring, page_size=page,
                                     n_splits=splits, **kw)
    else:
        kernels.attention_simt(q, out, cu, kvl, max_q_len=1, k_pages=kp.to(DEV), v_pages=vp.to(DEV),
                               page_table=pt.to(DEV), ring=ring, page_size=page, **kw)
    assert bool(torch.isfinite(out.float()).all()), "a place of the cache that was never written was read"
    for b, n in enumerate(lengths):
        if n > 1200:
            # too long for a matrix per head: the oracle's form for one query (the plain tests tie it to the other)
            ref = plain.attention_last_query(qs[b][0], ks[b], vs[b], n_q, n_kv, hd, scale, cap, window)
        else:
            # oracle over the whole sequence with the query as the last row
            qfull = torch.zeros(n, n_q * hd).to(dtype)
            qfull[-1] = qs[b][0]
            ref = _attention_oracle(qfull, ks[b], vs[b], n_q, n_kv, hd, scale, cap, window)[-1]
        close(out[b], ref, dtype, scale=float(ref.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,hd,window,cap", [(4, 2, 16, 8, 50.0), (6, 1, 32, 100, 20.0), (3, 3, 48, 0, 0.0),
                                                    (8, 4, 256, 0, 50.0), (8, 4, 256, 70, 50.0)])
def test_attention_paged(dtype, n_q, n_kv, hd, window, cap):
    _paged_case(dtype, n_q, n_kv, hd, window, cap, lengths=[1, 63, 64, 65, 129, 300], seed=hd + window)


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("n_q,n_kv,hd,window,cap", [(4, 2, 16, 8, 50.0), (6, 1, 32, 100, 20.0), (3, 3, 48, 0, 0.0),
                                                    (8, 4, 256, 0, 50.0), (8, 4, 256, 70, 50.0), (16, 1, 128, 0, 0.0),
                                                    (5, 1, 80, 200, 30.0)])
def test_attention_decode_tensor_cores(splits, n_q, n_kv, hd, window, cap):
    _paged_case(torch.bfloat16, n_q, n_kv, hd, window, cap, lengths=[1, 63, 64, 65, 129, 300, 1000],
                seed=hd + window, kernel="mma", splits=splits)


@pytest.mark.parametrize("splits", [17, 33, 40])
@pytest.mark.parametrize("n_q,n_kv,hd,window,cap", [(8, 4, 256, 0, 50.0), (8, 4, 256, 4096, 50.0), (32, 16, 128, 0, 50.0),
                                                    (6, 1, 32, 0, 20.0)])
def test_attention_decode_many_splits(splits, n_q, n_kv, hd, window, cap):
    """More splits than a warp has lanes (the merge then takes two rounds per thread), as one sequence of
    8,192 keys on four kv heads gets them (37 on 148 SMs); sequences of a few keys beside long ones leave
    most splits empty; with the real window the ring of 64 pages is read through 65 tiles."""
    _paged_case(torch.bfloat16, n_q, n_kv, hd, window, cap, lengths=[5300, 70, 2600, 4161], seed=hd + splits,
                kernel="mma", splits=splits)


def test_attention_decode_far_key_at_the_splits_of_one_long_sequence():
    """One sequence of 8,192 keys: the launch policy gives it 37 splits.  Key 17 carries all the weight."""
    n_q, n_kv, hd = 8, 4, 64
    splits = kernels.decode_splits(1, n_kv, 8192, 0, sms=148)
    assert splits == 37

    def special(qs, ks, vs):
        ks[0][17] = 0
        qs[0][:] = 0
        for g in range(n_kv):
            ks[0][17, g * hd] = 8.0
        for h in range(n_q):
            qs[0][0, h * hd] = 8.0
        vs[0][17] = 5.0

    _paged_case(torch.bfloat16, n_q, n_kv, hd, 0, 0.0, lengths=[8192], special=special, seed=3, kernel="mma",
                splits=splits)


def test_attention_decode_tensor_cores_skips_padding_rows():
    """A row with kv_len 0 is padding: its output is zero and the cache is not read for it."""
    n_q, n_kv, hd = 4, 2, 64
    kp = torch.randn(3, n_kv, 64, hd).to(torch.bfloat16).to(DEV)
    q = torch.randn(3, n_q * hd).to(torch.bfloat16).to(DEV)
    out = torch.full((3, n_q * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    pt = torch.tensor([[0, 1], [0, 0], [2, 0]], dtype=torch.int32, device=DEV)
    for splits in (1, 3):
        kernels.attention_decode_mma(q, out, torch.arange(4, dtype=torch.int32, device=DEV),
                                     torch.tensor([100, 0, 5], dtype=torch.int32, device=DEV), kp, kp, pt,
                                     ring=1 << 30, page_size=64, n_kv=n_kv, group=2, head_dim=hd, scale=0.1, cap=0.0,
                                     window=0, batch=3, n_splits=splits)
        assert float(out[1].float().abs().max()) == 0.0 and float(out[0].float().abs().max()) > 0


@pytest.mark.parametrize("dtype,kernel,splits", [(torch.float32, "simt", 1), (torch.bfloat16, "mma", 1),
                                                 (torch.bfloat16, "mma", 4)])
def test_attention_far_key_stands_out(dtype, kernel, splits):
    """One key hundreds of places back carries almost all the weight: a kernel
    that drops or misplaces a far page cannot pass."""
    n_q, n_kv, hd = 4, 2, 32
    far = 17

    def special(qs, ks, vs):
        for b in range(len(qs)):
            if ks[b].shape[0] <= far:
                continue
            ks[b][far] = 0
            qs[b][:] = 0
            for g in range(n_kv):
                ks[b][far, g * hd] = 8.0
            for h in range(n_q):
                qs[b][0, h * hd] = 8.0
            vs[b][far] = 5.0

    _paged_case(dtype, n_q, n_kv, hd, 0, 0.0, lengths=[400, 700, 18], special=special, seed=3, kernel=kernel,
                splits=splits)


@pytest.mark.parametrize("dtype,kernel,splits", [(torch.float32, "simt", 1), (torch.bfloat16, "mma", 1),
                                                 (torch.bfloat16, "mma", 3)])
def test_attention_window_edge(dtype, kernel, splits):
    """The key exactly `window` places back must be invisible, the one after it visible."""
    n_q, n_kv, hd, window = 2, 1, 16, 70

    def special(qs, ks, vs):
        for b in range(len(qs)):
            n = ks[b].shape[0]
            if n <= window:
                continue
            qs[b][:] = 0
            qs[b][0, 0] = 8.0
            qs[b][0, hd] = 8.0
            ks[b][n - 1 - window] = 0
            ks[b][n - 1 - window, 0] = 40.0      # just outside: would take all the weight if seen
            vs[b][n - 1 - window] = 1000.0
            ks[b][n - window] = 0
            ks[b][n - window, 0] = 6.0           # just inside
            vs[b][n - window] = 3.0

    _paged_case(dtype, n_q, n_kv, hd, window, 0.0, lengths=[71, 128, 129, 500], special=special, seed=4,
                kernel=kernel, splits=splits)


def test_attention_prompt_and_decode_agree_bitwise():
    """The float path gives the same bits for a query whether it runs in a prompt or as a decode step."""
    n_q, n_kv, hd, window, page = 4, 2, 32, 40, 64
    g = torch.Generator().manual_seed(9)
    n = 150
    qkv = torch.randn(n, (n_q + 2 * n_kv) * hd, generator=g).to(DEV)
    out = torch.empty(n, n_q * hd, device=DEV)
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    kw = dict(n_kv=n_kv, group=2, head_dim=hd, scale=0.2, cap=30.0, window=window)
    kernels.attention_simt(qkv[:, :n_q * hd], out, cu, torch.tensor([n], dtype=torch.int32, device=DEV), batch=1,
                           max_q_len=n, k=qkv[:, n_q * hd:(n_q + n_kv) * hd], v=qkv[:, (n_q + n_kv) * hd:], **kw)
    ring = 64
    kp = torch.zeros(1, n_kv, page, hd, device=DEV)
    vp = torch.zeros_like(kp)
    for p in range(n - ring, n):
        kp[0, :, p % ring, :] = qkv[p, n_q * hd:(n_q + n_kv) * hd].view(n_kv, hd)
        vp[0, :, p % ring, :] = qkv[p, (n_q + n_kv) * hd:].view(n_kv, hd)
    one = torch.empty(1, n_q * hd, device=DEV)
    kernels.attention_simt(qkv[n - 1:n, :n_q * hd].contiguous(), one, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                           torch.tensor([n], dtype=torch.int32, device=DEV), batch=1, max_q_len=1, k_pages=kp,
                           v_pages=vp, page_table=torch.zeros(1, 1, dtype=torch.int32, device=DEV), ring=ring,
                           page_size=page, **kw)
    assert torch.equal(one[0], out[n - 1])


def test_kernels_refuse_what_they_cannot_do():
    q = torch.zeros(2, 24, device=DEV)
    with pytest.raises(kernels.KernelError):
        kernels.attention_simt(q, torch.empty_like(q), torch.tensor([0, 2], dtype=torch.int32, device=DEV),
                               torch.tensor([2], dtype=torch.int32, device=DEV), n_kv=1, group=2, head_dim=12,
                               scale=1.0, cap=0.0, window=0, batch=1, max_q_len=2, k=q, v=q)
    with pytest.raises(kernels.KernelError):
        kernels.gated_act(torch.zeros(1, 8, device=DEV), torch.zeros(1, 4, device=DEV), "relu")
    with pytest.raises(kernels.KernelError):
        kernels.embed_scale(torch.zeros(1, dtype=torch.int32), torch.zeros(4, 4), 1.0, torch.zeros(1, 4))


@pytest.mark.parametrize("n_q,n_kv,hd,K,M", [(4, 2, 16, 64, 5), (6, 1, 32, 96, 3), (8, 4, 256, 2304, 8), (3, 1, 48, 72, 16),
                                             (5, 5, 64, 136, 9)])
def test_qkv_product_with_rotation_and_cache_write(n_q, n_kv, hd, K, M):
    """The few-token q/k/v product whose epilogue rotates q and k and writes k, v into the pages:
    against float64, with a padding row (nothing written) and a row that is not kept."""
    from brolm_b200 import kernels
    g = torch.Generator().manual_seed(hd * 7 + K)
    width, page, pages, half = (n_q + 2 * n_kv) * hd, 64, 4, hd // 2
    w = (torch.randn(width, K, generator=g) * 0.1).to(DEV).bfloat16()
    x = torch.randn(M, K, generator=g).to(DEV).bfloat16()
    pos_list = [3, 70, -1, 0, 129] + list(range(5, 16))
    row_list = [3, 64 + 6, 9, -1, 2 * 64 + 1] + list(range(200, 211))
    pos = torch.tensor(pos_list[:M], dtype=torch.int32, device=DEV)
    crow = torch.tensor(row_list[:M], dtype=torch.int32, device=DEV)
    ang = torch.arange(256, dtype=torch.float64)[:, None] * (10000.0 ** (-2.0 * torch.arange(half, dtype=torch.float64) / hd))
    table = torch.stack([ang.cos(), ang.sin()], -1).float().to(DEV).contiguous()
    for use_table, use_pages in ((True, True), (False, True), (True, False)):
        out = torch.full((M, width), 7.0, dtype=torch.bfloat16, device=DEV)
        k_pages = torch.zeros(pages, n_kv, page, hd, dtype=torch.bfloat16, device=DEV)
        v_pages = torch.zeros_like(k_pages)
        kernels.skinny_qkv_rope(x, w, out, pos, table if use_table else None, n_q, n_kv, hd,
                                k_pages if use_pages else None, v_pages if use_pages else None,
                                crow if use_pages else None, page)
        src = (x.double() @ w.double().t()).view(M, n_q + 2 * n_kv, hd)
        want = src.clone()
        if use_table:
            for t in range(M):
                p = pos_list[t]
                if p >= 0:
                    c, s = table[p, :, 0].double(), table[p, :, 1].double()
                    a, b = src[t, :n_q + n_kv, :half], src[t, :n_q + n_kv, half:]
                    want[t, :n_q + n_kv, :half] = a * c - b * s
                    want[t, :n_q + n_kv, half:] = a * s + b * c
        got = out.double().view(M, n_q + 2 * n_kv, hd)
        kept = set()
        for t in range(M):
            if pos_list[t] < 0:
                assert (got[t] == 7.0).all()
                continue
            err = (got[t] - want[t]).abs()
            assert (err <= 2.0 ** -8 * want[t].abs() + 1e-5 * want[t].abs().max()).all()      # one rounding
            r = row_list[t]
            if use_pages and r >= 0:
                kept.add(r)
                assert torch.equal(k_pages[r // page, :, r % page].double(), got[t, n_q:n_q + n_kv])
                assert torch.equal(v_pages[r // page, :, r % page].double(), got[t, n_q + n_kv:])
        mask = torch.ones(pages * page, dtype=torch.bool)
        mask[list(kept)] = False
        for pg in (k_pages, v_pages):
            assert (pg.permute(0, 2, 1, 3).reshape(pages * page, -1)[mask.to(DEV)] == 0).all()
