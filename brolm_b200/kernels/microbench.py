"""Times single kernels of brolm_b200 with CUDA events and prints what they reach.

    python -m brolm_b200.kernels.microbench attn_decode --batch 8 --ctx 8192 [--window 4096]
    python -m brolm_b200.kernels.microbench attn_prefill --tokens 2048
    python -m brolm_b200.kernels.microbench norms --batch 8
    python -m brolm_b200.kernels.microbench stream --batch 64            (the weight stream against the library)
    python -m brolm_b200.kernels.microbench timeline_decode --batch 8 --ctx 8192 --layers 6
    python -m brolm_b200.kernels.microbench timeline_prefill --tokens 2048 --layers 4

Sizes default to those of Gemma 2 2B (8 query heads, 4 kv heads of 256).  Inputs
are larger than the L2 cache or the L2 is flushed between repetitions.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import (attention_decode_mma, attention_prefill_mma, attention_prefill_tc, attention_prefill_tc_split, attention_tc_status, decode_splits, gemm_tc, gemm_tc_status, residual_rmsnorm,
               rmsnorm, skinny_gemm)

DEV = "cuda:0"


def timed(fn, reps: int, flush=None) -> float:
    """Median milliseconds of ``fn`` over ``reps`` runs, after three warm-up runs."""
    for _ in range(3):
        fn()
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]


def attn_decode(args) -> None:
    B, ctx, n_q, n_kv, hd = args.batch, args.ctx, args.heads, args.kv_heads, args.head_dim
    ring = (args.window + 63) // 64 * 64 if args.window else 1 << 30
    per_seq = min((ctx + 63) // 64, ring // 64)
    pages = B * per_seq
    kp = torch.randn(pages, n_kv, 64, hd, device=DEV).to(torch.bfloat16)
    vp = torch.randn(pages, n_kv, 64, hd, device=DEV).to(torch.bfloat16)
    table = torch.randperm(pages, device=DEV).int().view(B, per_seq).contiguous()
    q = torch.randn(B, n_q * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(q)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    kv_len = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
    if args.ragged:              # lengths spread evenly between a fifth of the context and all of it
        kv_len = torch.linspace(ctx / 5, ctx, B).round().int()[torch.randperm(B, generator=torch.Generator().manual_seed(1))].to(DEV)
    splits = args.splits or decode_splits(B, n_kv, ctx, args.window, ragged=args.ragged)
    n = B * n_q * splits
    scratch = (torch.empty(n * hd, dtype=torch.float32, device=DEV), torch.empty(n * 2, dtype=torch.float32, device=DEV))

    def run():
        attention_decode_mma(q, out, cu, kv_len, kp, vp, table, ring=ring, page_size=64, n_kv=n_kv, group=n_q // n_kv,
                             head_dim=hd, scale=1 / math.sqrt(hd), cap=50.0, window=args.window, batch=B,
                             n_splits=splits, scratch=scratch)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    ms = timed(run, args.reps, flush)
    keys = int(kv_len.clamp(max=args.window).sum()) if args.window else int(kv_len.sum())
    nbytes = keys * n_kv * hd * 2 * 2
    print(f"attn_decode batch={B} ctx={ctx}{' ragged' if args.ragged else ''} window={args.window} splits={splits}: {ms * 1e3:.1f} us, "
          f"{nbytes / ms / 1e6:.0f} GB/s of cache read")


def attn_prefill(args) -> None:
    T, n_q, n_kv, hd = args.tokens, args.heads, args.kv_heads, args.head_dim
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, device=DEV).to(torch.bfloat16)
    out = torch.empty(T, n_q * hd, dtype=torch.bfloat16, device=DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)

    def run():
        attention_prefill_mma(qkv[:, :n_q * hd], out, cu, qkv[:, n_q * hd:(n_q + n_kv) * hd],
                              qkv[:, (n_q + n_kv) * hd:], n_kv=n_kv, group=n_q // n_kv, head_dim=hd,
                              scale=1 / math.sqrt(hd), cap=args.cap, window=args.window, batch=1, max_q_len=T)

    # --splits: row blocks cut in two along their keys (0: the launcher's choice, -1: none)
    n_split = None if args.splits == 0 else max(0, args.splits)

    def run_tc():
        attention_prefill_tc(qkv[:, :n_q * hd], out, cu, qkv[:, n_q * hd:(n_q + n_kv) * hd],
                             qkv[:, (n_q + n_kv) * hd:], n_kv=n_kv, group=n_q // n_kv, head_dim=hd,
                             scale=1 / math.sqrt(hd), cap=args.cap, window=args.window, batch=1, max_q_len=T,
                             n_split=n_split)

    w = args.window or T
    keys = sum(min(p + 1, w) for p in range(T))
    flops = 4.0 * n_q * hd * keys
    for name, fn in (("tcgen05", run_tc), ("mma.sync", run)):
        ms = timed(fn, args.reps)
        cut = f" cut={attention_prefill_tc_split(T, n_kv, n_q // n_kv, args.window, 1) if n_split is None else n_split}" if fn is run_tc else ""
        print(f"attn_prefill {name} tokens={T} window={args.window}{cut}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.1f} TFLOP/s")
    print("attention_tc status", attention_tc_status())


def model_prefill(args) -> None:
    """One prompt through a model of Gemma 2 2B's layer sizes with few layers (for launch lists)."""
    import brolm_b200 as bb
    cfg = bb.Gemma2Config(num_hidden_layers=args.layers)
    model = bb.Model(cfg, dtype="bfloat16", device=DEV).init_random(seed=0, on_device=True)
    engine = bb.Engine(model, max_tokens=args.tokens + 64, max_slots=1)
    prompt = torch.randint(0, cfg.vocab_size, (args.tokens,), generator=torch.Generator().manual_seed(1)).tolist()

    def run():
        (s,) = engine.open(1)
        engine.step([s], [prompt])
        engine.close([s])

    ms = timed(run, args.reps)
    print(f"model_prefill layers={args.layers} tokens={args.tokens}: {ms:.3f} ms")


def skinny(args) -> None:
    """The few-token products of one Gemma 2 2B layer at --batch tokens (weights streamed once each)."""
    B, H, F = args.batch, args.hidden, args.inter
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    for name, n, k, epi in (("qkv", qkv, H, "store"), ("o", H, args.heads * args.head_dim, "store"),
                            ("gate_up+act", F, H, "gated"), ("down", H, F, "store")):
        x = torch.randn(B, k, device=DEV).to(torch.bfloat16)
        w = torch.randn(2 * n if epi == "gated" else n, k, device=DEV).to(torch.bfloat16)
        out = torch.empty(B, n, dtype=torch.bfloat16, device=DEV)
        ms = timed(lambda: skinny_gemm(x, w, out, epi), args.reps, flush)
        print(f"skinny {name} rows={B} N={w.shape[0]} K={k}: {ms * 1e3:.1f} us, {w.numel() * 2 / ms / 1e6:.0f} GB/s of weights")


def stream(args) -> None:
    """The products of one layer at --batch tokens (17 to 128): the tcgen05 weight stream against the library."""
    from . import gemm_stream, gemm_stream_parts, gemm_stream_status
    B, H, F = args.batch, args.hidden, args.inter
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    total_own = total_lib = 0.0
    for name, n, k, epi in (("qkv", qkv, H, "store"), ("o", H, args.heads * args.head_dim, "parts"),
                            ("gate_up+act", F, H, "gated"), ("down", H, F, "parts")):
        x = torch.randn(B, k, device=DEV).to(torch.bfloat16)
        rows = 2 * n if epi == "gated" else n
        w = torch.randn(rows, k, device=DEV).to(torch.bfloat16)
        parts = gemm_stream_parts(x, w) if epi == "parts" else 1
        out = (torch.empty(parts, B, n, dtype=torch.float32, device=DEV) if parts > 1 else
               torch.empty(B, n, dtype=torch.float32 if epi == "parts" else torch.bfloat16, device=DEV))
        wide = torch.empty(B, rows, dtype=torch.bfloat16, device=DEV)
        own = timed(lambda: gemm_stream(x, w, out, "gated" if epi == "gated" else "store"), args.reps, flush)
        lib = timed(lambda: torch.mm(x, w.t(), out=wide), args.reps, flush)
        total_own += own
        total_lib += lib
        print(f"gemm_stream {name} rows={B} N={rows} K={k} slices={parts}: {own * 1e3:.1f} us, "
              f"{w.numel() * 2 / own / 1e6:.0f} GB/s of weights (library product alone: {lib * 1e3:.1f} us, "
              f"{w.numel() * 2 / lib / 1e6:.0f} GB/s)")
    print(f"one layer: {total_own * 1e3:.1f} us own, {total_lib * 1e3:.1f} us library; status {gemm_stream_status()}")


def gemm(args) -> None:
    """The many-token products of one Gemma 2 2B layer at --tokens tokens on tcgen05, against the library."""
    T, H, F = args.tokens, args.hidden, args.inter
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    for name, n, k, epi in (("qkv", qkv, H, "store"), ("o", H, args.heads * args.head_dim, "store"),
                            ("gate_up+act", F, H, "gated"), ("down", H, F, "store")):
        x = torch.randn(T, k, device=DEV).to(torch.bfloat16)
        rows = 2 * n if epi == "gated" else n
        w = torch.randn(rows, k, device=DEV).to(torch.bfloat16)
        out = torch.empty(T, n, dtype=torch.bfloat16, device=DEV)
        wide = torch.empty(T, rows, dtype=torch.bfloat16, device=DEV)
        ms = timed(lambda: gemm_tc(x, w, out, epi), args.reps)
        one = timed(lambda: gemm_tc(x, w, out, epi, pairs=False), args.reps)
        lib = timed(lambda: torch.mm(x, w.t(), out=wide), args.reps)
        fl = 2.0 * T * rows * k
        print(f"gemm_tc {name} M={T} N={rows} K={k}: pairs of SMs {ms * 1e3:.1f} us, {fl / ms / 1e9:.0f} TFLOP/s; "
              f"one block per tile {one * 1e3:.1f} us, {fl / one / 1e9:.0f} TFLOP/s "
              f"(library product alone, without the activation: {lib * 1e3:.1f} us, {fl / lib / 1e9:.0f} TFLOP/s)")
    print("gemm_tc status", gemm_tc_status())


def norms(args) -> None:
    B, H = args.batch, args.hidden
    h = torch.randn(B, H, device=DEV)
    y = torch.randn(B, H, device=DEV)
    w = torch.randn(H, device=DEV).to(torch.bfloat16)
    out = torch.empty(B, H, dtype=torch.bfloat16, device=DEV)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    ms = timed(lambda: residual_rmsnorm(h, y, w, 1e-6, 1.0, w, 1e-6, 1.0, out), args.reps, flush)
    print(f"residual_rmsnorm rows={B} hidden={H}: {ms * 1e3:.1f} us")
    ms = timed(lambda: rmsnorm(h, w, 1e-6, 1.0, out), args.reps, flush)
    print(f"rmsnorm rows={B} hidden={H}: {ms * 1e3:.1f} us")


def _config(args):
    """The Gemma 2 configuration of --layers layers with the layer sizes given on the command line
    (the defaults are those of Gemma 2 2B)."""
    import brolm_b200 as bb
    return bb.Gemma2Config(num_hidden_layers=args.layers, hidden_size=args.hidden, intermediate_size=args.inter,
                           num_attention_heads=args.heads, num_key_value_heads=args.kv_heads, head_dim=args.head_dim,
                           query_pre_attn_scalar=float(args.scalar or args.head_dim))


def _print_timeline(events, first: int, title: str) -> None:
    ev = events[first:]
    t0 = ev[0].time_range.start
    prev_end = t0
    print(title)
    print("   start     time  gap to the end of all kernels before   kernel (microseconds)")
    for e in ev:
        start, dur = e.time_range.start - t0, e.time_range.end - e.time_range.start
        name = e.name.replace("void ", "").replace("(anonymous namespace)::", "").replace("<unnamed>::", "")[:64]
        print(f"{start:8.2f} {dur:8.2f} {e.time_range.start - prev_end:8.2f}  {name}")
        prev_end = max(prev_end, e.time_range.end)
    print(f"total {prev_end - t0:.1f} us")


def _cuda_events(fn):
    """Device activity records (CUPTI, through torch.profiler) of what ``fn`` launches: every kernel with its
    start and end on the device's own clock, captured steps included.  Unlike ncu nothing is serialised, so
    the overlap of kernels launched with programmatic stream serialization shows (negative gaps); the
    records cost a little time per kernel, so the figures are for comparing shares, not for quoting."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        fn()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    ev.sort(key=lambda e: e.time_range.start)
    return ev


def timeline_decode(args) -> None:
    """One captured decode step of a model of Gemma 2 2B's layer sizes (--layers of them), kernel by kernel."""
    import brolm_b200 as bb
    B, ctx = args.batch, args.ctx
    cfg = _config(args)
    model = bb.Model(cfg, dtype="bfloat16", device=DEV).init_random(seed=0, on_device=True)
    eng = bb.Engine(model, max_tokens=B * ((ctx + 63) // 64 * 64), max_slots=B, max_seq_len=ctx)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (ctx - 40,), generator=g).tolist() for _ in range(B)]
    slots = eng.open(B)
    sampler = bb.Sampler(bb.SamplingParams(temperature=0.0))
    streams = torch.arange(B, dtype=torch.int32, device=DEV)
    ids = sampler(eng.step(slots, prompts), streams, 0)
    pick = list(range(B))
    state = {"ids": ids, "n": 1}

    def steps(n):
        for _ in range(n):
            state["ids"] = sampler(eng.step_from(slots, state["ids"], pick), streams, state["n"])
            state["n"] += 1

    steps(20)
    torch.cuda.synchronize()
    ev = _cuda_events(lambda: steps(3))
    first = [i for i, e in enumerate(ev) if "embed" in e.name][-1]
    _print_timeline(ev, first, f"decode step, batch {B}, context {ctx}, {args.layers} layers, hidden {args.hidden}")


def timeline_prefill(args) -> None:
    """One prompt of --tokens tokens through --layers layers of the Gemma 2 2B sizes, kernel by kernel."""
    import brolm_b200 as bb
    cfg = _config(args)
    model = bb.Model(cfg, dtype="bfloat16", device=DEV).init_random(seed=0, on_device=True)
    eng = bb.Engine(model, max_tokens=args.tokens + 64, max_slots=1)
    prompt = torch.randint(0, cfg.vocab_size, (args.tokens,), generator=torch.Generator().manual_seed(1)).tolist()

    def run():
        (s,) = eng.open(1)
        eng.step([s], [prompt])
        eng.close([s])

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    ev = _cuda_events(run)
    _print_timeline(ev, 0, f"prompt of {args.tokens} tokens, {args.layers} layers, hidden {args.hidden}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["attn_decode", "attn_prefill", "model_prefill", "norms", "skinny", "gemm", "stream",
                                     "timeline_decode", "timeline_prefill"])
    ap.add_argument("--inter", type=int, default=9216)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=256)
    ap.add_argument("--hidden", type=int, default=2304)
    ap.add_argument("--scalar", type=float, default=0.0, help="query_pre_attn_scalar (0: head_dim)")
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--ragged", action="store_true", help="attn_decode: sequences of unequal lengths up to --ctx")
    ap.add_argument("--cap", type=float, default=50.0, help="soft cap of the attention scores (0: none)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--no-tc", action="store_true", help="many-token products through the library instead of gemm_tc")
    args = ap.parse_args()
    if args.no_tc:
        from .. import kernels
        kernels.USE_TC_GEMM = False
    {"attn_decode": attn_decode, "attn_prefill": attn_prefill, "model_prefill": model_prefill,
     "norms": norms, "skinny": skinny, "gemm": gemm, "stream": stream,
     "timeline_decode": timeline_decode, "timeline_prefill": timeline_prefill}[args.what](args)


if __name__ == "__main__":
    main()
