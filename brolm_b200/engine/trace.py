"""Trace replay: given token ids step by step, write the logits.

One JSON object per line on the input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

A request seen for the first time takes a slot; its later entries go on by one
token; a request named in ``end`` gives its slot and pages back after the
step.  For a step in which something is wanted, ``<out>/<step>.f32`` holds
the logits at the wanted places, in the order of the entries and of ``want``,
as little-endian float32 [wanted, vocab].  After every step ``done <step>`` is
printed and flushed.  Nothing is sampled, and there is no model code here:
the replay drives the same ``Engine.step`` that generation uses.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO

import numpy as np

from .model import load_model
from .step import Engine


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines: IO[str], device: str = "cuda:0",
           log: IO[str] = sys.stdout) -> None:
    os.makedirs(out_dir, exist_ok=True)
    model = load_model(model_dir, dtype=dtype, device=device)
    engine = Engine(model, max_tokens=max_tokens)
    slot_of: dict[str, int] = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = rec.get("entries", [])
        if entries:
            fresh = [str(e["id"]) for e in entries if str(e["id"]) not in slot_of]
            for rid, slot in zip(fresh, engine.open(len(fresh))):
                slot_of[rid] = slot
            slots = [slot_of[str(e["id"])] for e in entries]
            want = [list(e.get("want", [])) for e in entries]
            logits = engine.step(slots, [e["tokens"] for e in entries], want)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                with open(os.path.join(out_dir, f"{step}.f32"), "wb") as fh:
                    fh.write(np.ascontiguousarray(arr).tobytes())
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slot_of:
                engine.close([slot_of.pop(rid)])
        print(f"done {step}", file=log, flush=True)


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="Feed given token ids through a model step by "
                                 "step and write the logits at the wanted places.")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", required=True, type=int,
                    help="most tokens live requests hold at one time (each rounded up to a multiple of 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, args.device)
    return 0
