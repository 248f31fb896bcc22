#!/usr/bin/env python3
"""Decode and prefill throughput of brolm_b200 on one B200, one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--context C] [--layers L]

The default run has the layer sizes of Gemma 2 2B with random bfloat16
weights, a batch of 8 and a context of 8192 tokens.  A step is one decode
step of the whole batch.  ``value`` is decoded tokens a second, timed on the
device; ``e2e`` is the same through ``brolm_b200.generate`` with host tokens
in and out; ``prefill`` is one prompt of 2,048 tokens; ``points`` holds
decoding at batch 1 and 64.  More than one GPU is not what this library does:
``--gpus N`` with N > 1 says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            raw = json.load(fh)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw.get("bf16_tflops_sustained")
                                                                     or raw["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


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


def decode_bytes(cfg, layers: int, batch: int, context: int, itemsize: int = 2) -> float:
    """Bytes a decode step has to read: every weight once and the cache of the live requests."""
    H, F = cfg.hidden_size, cfg.intermediate_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * F * H + 4 * H
    weights = (layers * per_layer + cfg.vocab_size * H + H) * itemsize
    kv = 0
    for i in range(layers):
        keys = min(context, cfg.sliding_window) if cfg.is_sliding(i) else context
        kv += batch * keys * 2 * cfg.kv_dim * itemsize
    return float(weights + kv)


def prefill_flops(cfg, layers: int, tokens: int) -> float:
    H, F = cfg.hidden_size, cfg.intermediate_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * F * H
    linear = 2.0 * tokens * per_layer * layers
    attn = 0.0
    for i in range(layers):
        w = cfg.sliding_window if cfg.is_sliding(i) else tokens
        keys = sum(min(p + 1, w) for p in range(tokens))
        attn += 4.0 * cfg.q_dim * keys
    return linear + attn + 2.0 * cfg.vocab_size * H


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="brolm_b200")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "wlejon/brolm is a C++ project without a Python "
                          "package (pip: neither setup.py nor pyproject.toml) and needs the absent sibling library "
                          "brotensor to build; it also has no batched Gemma 2 decode to time"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: brolm_b200 is a one-GPU library; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    import brolm_b200 as bb
    from brolm_b200 import kernels

    pk = peaks()
    cfg = bb.Gemma2Config()                      # the 2B sizes are the configuration's defaults
    full_layers = cfg.num_hidden_layers
    if args.layers:
        cfg.num_hidden_layers = args.layers
    layers = cfg.num_hidden_layers
    dev = "cuda:0"
    torch.cuda.set_device(0)
    model = bb.Model(cfg, dtype="bfloat16", device=dev).init_random(seed=0, on_device=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # larger than the 126 MB L2

    def decode_run(batch: int, context: int, steps: int, warmup: int):
        """Decode ``steps`` tokens per sequence after ``warmup`` untimed ones, ending at ``context`` tokens.

        A step reads every weight and the live cache once, gigabytes against an L2 of 126 MB, so
        nothing of one step is still cached for the next and no flush is put between steps.
        Two passes over the same prompts.  End to end: ``brolm_b200.generate`` with host token ids in and
        out; every step copies the step's tokens from pinned host memory to the device and reads the
        sampled ids back.  Device: the same steps fed with the tokens the first pass produced, queued
        without reading anything back, timed with CUDA events."""
        warmup += SETTLE
        total = steps + warmup
        prompt_len = context - total - 1
        engine = bb.Engine(model, max_tokens=batch * ((context + 63) // 64 * 64), max_slots=batch,
                           max_seq_len=context)
        g = torch.Generator().manual_seed(42)
        prompts = [torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist() for _ in range(batch)]
        opts = bb.GenerateOptions(max_new_tokens=total + 1, sampling=bb.SamplingParams(temperature=0.0),
                                  stop_on_eos=False)
        stamps: list[float] = []

        def on_step(produced: int, active: int) -> None:
            # called after the step's tokens reached the host
            stamps.append(time.perf_counter())

        with ClockSampler() as clocks:
            out = bb.generate(engine, prompts, eos_id=-1, opts=opts, on_step=on_step)
            torch.cuda.synchronize()
            assert all(len(o) == total + 1 for o in out)
            # on_step 0 follows the prefill; steps 1..warmup are warm-up; the rest are timed
            e2e_s = stamps[warmup + steps] - stamps[warmup]

            # device pass: the same tokens, nothing read back
            sampler = bb.Sampler(opts.sampling)
            streams = torch.arange(batch, dtype=torch.int32, device=dev)
            slots = engine.open(batch)
            engine.step(slots, prompts)
            events = []
            launches = []
            for i in range(total):
                if i >= warmup:
                    ev = torch.cuda.Event(enable_timing=True)
                    ev.record()
                    events.append(ev)
                    launches.append(kernels.launch_count())
                logits = engine.step(slots, [[o[i]] for o in out])
                sampler(logits, streams, i + 1)
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            events.append(ev)
            launches.append(kernels.launch_count())
            torch.cuda.synchronize()
            engine.close(slots)
        ms = events[0].elapsed_time(events[-1]) / steps
        return {"tok_s": batch * 1000.0 / ms, "ms": ms, "e2e_tok_s": batch * steps / e2e_s,
                "launches": launches[-1] - launches[0], "clocks": clocks.summary(),
                "h2d": engine.last_h2d_bytes, "d2h": 4 * batch}

    main_run = decode_run(args.batch, args.context, args.steps, args.warmup)
    bytes_step = decode_bytes(cfg, layers, args.batch, args.context)
    achieved = bytes_step / (main_run["ms"] * 1e-3) / 1e9

    result = {
        "metric": "decode tokens/s (Gemma 2 2B sizes, batch 8, context 8192)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
        "impl": "brolm_b200",
        "config": {"model": "gemma-2-2b sizes", "layers": layers, "layers_of_configuration": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "sliding_window": cfg.sliding_window, "global_batch": args.batch, "seq_len": args.context,
                   "parallelism": "none (1 GPU)", "settle_steps": SETTLE,
                   "l2": f"inputs larger than L2 ({bytes_step / 1e9:.1f} GB read per step)",
                   "peaks": pk["source"]},
        "clocks": main_run["clocks"],
        "e2e": {"value": round(main_run["e2e_tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": main_run["h2d"],
                "d2h_bytes_per_step": main_run["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
    }

    if not args.no_points:
        points = {}
        for b in (1, 64):
            r = decode_run(b, args.context, max(8, args.steps // 4), 3)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
        # the workload of the configuration's own description: prompts of 1,024 tokens, 256 generated
        for b in (1, 8, 64):
            r = decode_run(b, 1024 + 256, max(8, args.steps // 2), 3)
            points[f"decode_b{b}_ctx1280"] = round(r["tok_s"], 1)
        result["points"] = points
        # prefill of 2,048 tokens, one sequence, logits of the last token
        T = 2048
        engine = bb.Engine(model, max_tokens=T + 64, max_slots=1)
        prompt = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(1)).tolist()
        times = []
        for it in range(3 + 3):
            (s,) = engine.open(1)
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([s], [prompt])
            e1.record()
            torch.cuda.synchronize()
            engine.close([s])
            if it >= 3:
                times.append(e0.elapsed_time(e1))
        ms = sorted(times)[len(times) // 2]
        fl = prefill_flops(cfg, layers, T)
        result["prefill"] = {"value": round(T * 1000.0 / ms, 1), "tokens": T, "ms": round(ms, 3),
                             "frac": round(fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk["source"]}
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
