#!/usr/bin/env python3
"""Decode and prefill throughput of brolm_b200 on one B200, one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--size 2b|9b|27b] [--batch B] [--context C] [--layers L]

The default run (``--size 2b``) has the layer sizes of Gemma 2 2B with random
bfloat16 weights, a batch of 8 and a context of 8192 tokens.  A step is one
decode step of the whole batch.  ``value`` is decoded tokens a second, timed on
the device: the median of ``repeats`` timed regions of exactly K steps each;
``e2e`` is the same through ``brolm_b200.generate`` with host tokens in and
out; ``prefill`` is one prompt of 2,048 tokens; ``points`` holds decoding at
batch 1 and 64, ``points_roofline`` their fractions of the memory's rate.

``--size 9b``: Gemma 2 9B sizes, 16 prompts of 128 to 6,144 tokens (seeded) in
one prefill step, then decode steps of the 16 sequences (K defaults to 128).
``--size 27b``: Gemma 2 27B sizes, a prompt of 2,048 tokens and decoding at
batch 8 (headline) and batch 1 (a point).  Same JSON shape.

More than one GPU is not what this library does: ``--gpus N`` with N > 1 says
so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The layer sizes of the three workloads (the keys of Gemma 2's config.json; 2B is the configuration's default).
SIZES = {
    "2b": dict(),
    "9b": dict(num_hidden_layers=42, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8, head_dim=256,
               intermediate_size=14336, query_pre_attn_scalar=256.0),
    "27b": dict(num_hidden_layers=46, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                intermediate_size=36864, query_pre_attn_scalar=144.0),
}
REPEATS = 3


def peaks() -> dict:
    """The roofline's denominators: measured on this pool when the file is there, else the fallback.
    ``bf16_burst`` is the product peak of a kernel timed alone (what the prompt's fraction is taken
    against: the prompt is timed alone, between synchronisations and after an L2 flush);
    ``bf16_sustained`` the peak of a seconds-long loop under the power cap."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            raw = json.load(fh)
        burst = float(raw["bf16_tflops"])
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_burst": burst,
                "bf16_sustained": float(raw.get("bf16_tflops_sustained") or burst), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (read only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# Decode steps that every run puts between its prompt and its warm-up steps.  The prompt (batch x
# context tokens at full compute power) leaves the GPU with lowered clocks for some tens of
# milliseconds: the first 10-30 decode steps after it take up to 1.4 times as long as the steady
# ones that the metric is about (measured: 3.4, then 2.8, then 2.45 ms at batch 8, context 8192).
SETTLE = 32


def decode_bytes(cfg, layers: int, lengths, itemsize: int = 2) -> float:
    """Bytes a decode step has to read: every weight once and the cache of the live requests,
    ``lengths`` being the tokens each of them holds (a windowed layer holds at most its window)."""
    if isinstance(lengths, tuple) and len(lengths) == 2:         # (batch, context): equal lengths
        lengths = [lengths[1]] * lengths[0]
    H, F = cfg.hidden_size, cfg.intermediate_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * F * H + 4 * H
    weights = (layers * per_layer + cfg.vocab_size * H + H) * itemsize
    kv = 0.0
    for i in range(layers):
        for n in lengths:
            keys = min(n, cfg.sliding_window) if cfg.is_sliding(i) else n
            kv += keys * 2 * cfg.kv_dim * itemsize
    return float(weights + kv)


def prefill_flops(cfg, layers: int, tokens) -> float:
    """Floating-point operations of one prefill step; ``tokens``: a prompt length or a list of them."""
    lengths = [tokens] if isinstance(tokens, int) else list(tokens)
    H, F = cfg.hidden_size, cfg.intermediate_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * F * H
    linear = 2.0 * sum(lengths) * per_layer * layers
    attn = 0.0
    for i in range(layers):
        for n in lengths:
            w = cfg.sliding_window if cfg.is_sliding(i) else n
            full = min(n, w)
            keys = full * (full + 1) // 2 + (n - full) * w          # sum over positions of min(p + 1, w)
            attn += 4.0 * cfg.q_dim * keys
    return linear + attn + 2.0 * cfg.vocab_size * H * len(lengths)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps in a timed region (default 64; 128 for 9b)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="brolm_b200")
    ap.add_argument("--size", default="2b", choices=sorted(SIZES))
    ap.add_argument("--batch", type=int, default=0, help="sequences of the headline run (default: the workload's)")
    ap.add_argument("--context", type=int, default=0,
                    help="tokens a sequence holds after the last timed step (default 8192; 2304 for 27b)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--repeats", type=int, default=REPEATS, help="timed regions of K steps each; value = their median")
    ap.add_argument("--no-points", action="store_true", help="skip the other batch sizes and the prefill measurement")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "wlejon/brolm is a C++ project without a Python "
                          "package (pip: neither setup.py nor pyproject.toml) and needs the absent sibling library "
                          "brotensor to build; it also has no batched Gemma 2 decode to time"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: brolm_b200 is a one-GPU library; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    steps = args.steps or (128 if args.size == "9b" else 64)
    context = args.context or (2048 + 256 if args.size == "27b" else 8192)

    import torch

    import brolm_b200 as bb
    from brolm_b200 import kernels

    pk = peaks()
    cfg = bb.Gemma2Config(**SIZES[args.size])
    full_layers = cfg.num_hidden_layers
    if args.layers:
        cfg.num_hidden_layers = args.layers
    layers = cfg.num_hidden_layers
    dev = "cuda:0"
    torch.cuda.set_device(0)
    model = bb.Model(cfg, dtype="bfloat16", device=dev).init_random(seed=0, on_device=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # larger than the 126 MB L2

    def decode_run(prompt_lengths, steps: int, warmup: int, repeats: int, e2e: bool):
        """Decode after one prefill step of prompts of ``prompt_lengths``: SETTLE + ``warmup`` untimed
        steps, then ``repeats`` timed regions of ``steps`` steps each.

        A step reads every weight and the live cache once, gigabytes against an L2 of 126 MB, so
        nothing of one step is still cached for the next and no flush is put between steps.
        Device timing: the generation loop's own steps (``Engine.step_from``: the ids a step's sampler
        drew feed the next step on the device), queued without reading anything back, CUDA events
        around each region.  End to end (``e2e``): ``brolm_b200.generate`` with host token ids in and
        out; every step copies its description from pinned host memory to the device and reads the
        sampled ids back; host clock between the callbacks that follow those reads."""
        batch = len(prompt_lengths)
        warmup += SETTLE
        total = warmup + repeats * steps
        longest = max(prompt_lengths) + total + 1
        need = sum((n + total + 1 + 63) // 64 * 64 for n in prompt_lengths)
        engine = bb.Engine(model, max_tokens=need, max_slots=batch, max_seq_len=longest)
        g = torch.Generator().manual_seed(42)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in prompt_lengths]
        opts = bb.GenerateOptions(max_new_tokens=total + 1, sampling=bb.SamplingParams(temperature=0.0),
                                  stop_on_eos=False)
        e2e_tok_s = None
        with ClockSampler() as clocks:
            if e2e:
                stamps: list[float] = []
                # called after each step's tokens reached the host; call 0 follows the prefill
                out = bb.generate(engine, prompts, eos_id=-1, opts=opts,
                                  on_step=lambda produced, active: stamps.append(time.perf_counter()))
                torch.cuda.synchronize()
                assert all(len(o) == total + 1 for o in out)
                rates = [batch * steps / (stamps[warmup + (r + 1) * steps] - stamps[warmup + r * steps])
                         for r in range(repeats)]
                e2e_tok_s = statistics.median(rates)

            sampler = bb.Sampler(opts.sampling)
            streams = torch.arange(batch, dtype=torch.int32, device=dev)
            pick = list(range(batch))
            slots = engine.open(batch)
            logits = engine.step(slots, prompts)
            ids = sampler(logits, streams, 0)
            marks, launches = [], []
            for i in range(total):
                if i >= warmup and (i - warmup) % steps == 0:
                    ev = torch.cuda.Event(enable_timing=True)
                    ev.record()
                    marks.append(ev)
                    launches.append(kernels.launch_count())
                logits = engine.step_from(slots, ids, pick)
                ids = sampler(logits, streams, i + 1)
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append(ev)
            launches.append(kernels.launch_count())
            torch.cuda.synchronize()
            engine.close(slots)
        region_ms = [marks[r].elapsed_time(marks[r + 1]) / steps for r in range(repeats)]
        # what each region had to read: the lengths at its middle step
        region_bytes = [decode_bytes(cfg, layers, [n + 1 + warmup + r * steps + steps // 2 for n in prompt_lengths])
                        for r in range(repeats)]
        gbs = [b / (ms * 1e-3) / 1e9 for b, ms in zip(region_bytes, region_ms)]
        ms = statistics.median(region_ms)
        return {"tok_s": batch * 1000.0 / ms, "ms": ms, "best_tok_s": batch * 1000.0 / min(region_ms),
                "e2e_tok_s": e2e_tok_s, "launches": launches[1] - launches[0], "clocks": clocks.summary(),
                "h2d": engine.last_h2d_bytes, "d2h": 4 * batch, "gbs": statistics.median(gbs),
                "bytes": statistics.median(region_bytes), "final": [n + total + 1 for n in prompt_lengths]}

    def equal_prompts(batch: int, context: int, steps: int, warmup: int, repeats: int):
        """Prompts such that the last timed step ends at ``context`` tokens."""
        return [context - (SETTLE + warmup + repeats * steps) - 1] * batch

    def prefill_run(lengths):
        """One prefill step of prompts of ``lengths`` (logits of each last token), the median of three
        after three untimed ones, the L2 flushed before each."""
        need = sum((n + 63) // 64 * 64 for n in lengths) + 64
        engine = bb.Engine(model, max_tokens=need, max_slots=len(lengths), max_seq_len=max(lengths) + 1)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lengths]
        times = []
        for it in range(3 + 3):
            slots = engine.open(len(lengths))
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step(slots, prompts)
            e1.record()
            torch.cuda.synchronize()
            engine.close(slots)
            if it >= 3:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        fl = prefill_flops(cfg, layers, list(lengths))
        T = sum(lengths)
        return {"value": round(T * 1000.0 / ms, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(fl / (ms * 1e-3) / (pk["bf16_burst"] * 1e12), 4),
                "frac_sustained": round(fl / (ms * 1e-3) / (pk["bf16_sustained"] * 1e12), 4),
                "tflops": round(fl / (ms * 1e-3) / 1e12, 1), "peak": pk["bf16_burst"],
                "of": f"{pk['source']} bf16 burst peak (the step is timed alone after an L2 flush)"}

    if args.size == "9b":
        g = torch.Generator().manual_seed(9)
        prompt_lengths = torch.randint(128, 6144 + 1, (args.batch or 16,), generator=g).tolist()
        what = f"{len(prompt_lengths)} prompts of 128 to 6144 tokens"
    else:
        batch = args.batch or 8
        prompt_lengths = equal_prompts(batch, context, steps, args.warmup, args.repeats)
        what = f"batch {batch}, context {context}"
    main_run = decode_run(prompt_lengths, steps, args.warmup, args.repeats, e2e=True)
    name = {"2b": "Gemma 2 2B", "9b": "Gemma 2 9B", "27b": "Gemma 2 27B"}[args.size]

    result = {
        "metric": f"decode tokens/s ({name} sizes, {what})",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
        "impl": "brolm_b200",
        "config": {"model": f"gemma-2-{args.size} sizes", "layers": layers, "layers_of_configuration": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "sliding_window": cfg.sliding_window, "global_batch": len(prompt_lengths),
                   "seq_len": max(main_run["final"]), "seq_len_min": min(main_run["final"]),
                   "parallelism": "none (1 GPU)", "settle_steps": SETTLE, "repeats": args.repeats,
                   "l2": f"inputs larger than L2 ({main_run['bytes'] / 1e9:.1f} GB read per step)",
                   "peaks": pk["source"]},
        "clocks": main_run["clocks"],
        "repeats": {"n": args.repeats, "median": round(main_run["tok_s"], 1), "best": round(main_run["best_tok_s"], 1)},
        "e2e": {"value": round(main_run["e2e_tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": main_run["h2d"],
                "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(main_run["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_run["gbs"] / pk["hbm_gbs"], 4), "of": pk["source"]},
    }

    if not args.no_points:
        points, fracs, best = {}, {}, {}

        def point(key: str, lengths, k: int) -> None:
            r = decode_run(lengths, k, 3, args.repeats, e2e=False)
            points[key] = round(r["tok_s"], 1)
            best[key] = round(r["best_tok_s"], 1)
            fracs[key] = round(r["gbs"] / pk["hbm_gbs"], 4)

        if args.size == "2b":
            for b in (1, 64):
                point(f"decode_b{b}", equal_prompts(b, context, 64, 3, args.repeats), 64)
            # the workload of the configuration's own description: prompts of 1,024 tokens, 256 generated
            for b in (1, 8, 64):
                point(f"decode_b{b}_ctx1280", equal_prompts(b, 1024 + 256, 64, 3, args.repeats), 64)
        elif args.size == "27b":
            # prompts of 2,048 tokens, 256 generated
            point("decode_b1", equal_prompts(1, context, 64, 3, args.repeats), 64)
        result["points"] = points
        result["points_best"] = best
        result["points_roofline"] = fracs
        result["prefill"] = prefill_run(prompt_lengths if args.size == "9b" else [2048])
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
