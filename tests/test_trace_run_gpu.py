"""bin/trace_run as a user runs it: the same requests whole, with the last 32
tokens one by one, and in batches of unequal lengths, in both element types,
compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.helpers import make_folder, oracle_inputs, random_prompts
from tests.plain import gemma2_plain as plain
from tests.test_engine_gpu import STORE, TOL

pytestmark = pytest.mark.gpu
ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def run_trace(folder, dtype, out, max_tokens, steps):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out, "--max-tokens", str(max_tokens)], input=text, capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]


def read(out, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_three_ways(tmp_path, name, dtype):
    folder = make_folder(tmp_path, name, STORE[dtype])
    config, weights = oracle_inputs(folder)
    V = config["vocab_size"]
    reqs = random_prompts(V, [40, 100, 7, 130], seed=61)
    refs = [plain.forward(config, weights, p) for p in reqs]
    tol = TOL[dtype]

    # (1) whole, one after another, every position wanted
    steps = [{"step": i, "entries": [{"id": f"r{i}", "tokens": p, "want": list(range(len(p)))}], "end": [f"r{i}"]}
             for i, p in enumerate(reqs)]
    out = str(tmp_path / "whole")
    run_trace(folder, dtype, out, 192, steps)          # room for the longest request only: slots are reused
    def near(got, ref):
        return float((got.double() - ref).abs().max()) <= tol * float(ref.abs().max())

    for i, r in enumerate(refs):
        assert near(read(out, i, V), r)

    # (2) the last 32 tokens one by one
    steps, expect, n = [], {}, 0
    for i, p in enumerate(reqs):
        k = max(len(p) - 32, 1)
        steps.append({"step": n, "entries": [{"id": i, "tokens": p[:k], "want": [k - 1]}], "end": []})
        expect[n] = refs[i][k - 1:k]
        n += 1
        for j in range(k, len(p)):
            steps.append({"step": n, "entries": [{"id": i, "tokens": [p[j]], "want": [0]}],
                          "end": [i] if j == len(p) - 1 else []})
            expect[n] = refs[i][j:j + 1]
            n += 1
    out = str(tmp_path / "tail")
    run_trace(folder, dtype, out, 192, steps)
    for s, r in expect.items():
        assert near(read(out, s, V), r)

    # (3) one batch of unequal lengths; shorter requests end earlier; then a second batch on the same cache
    def batch_steps(ids, first_step):
        steps, expect = [], {}
        pre = {i: max(1, len(reqs[i]) // 2) for i in ids}
        steps.append({"step": first_step, "entries": [{"id": f"b{first_step}_{i}", "tokens": reqs[i][:pre[i]],
                                                      "want": [pre[i] - 1]} for i in ids],
                      "end": [f"b{first_step}_{i}" for i in ids if pre[i] == len(reqs[i])]})
        expect[first_step] = torch.cat([refs[i][pre[i] - 1:pre[i]] for i in ids])
        done = dict(pre)
        live = [i for i in ids if done[i] < len(reqs[i])]
        s = first_step + 1
        while live:
            ending = [i for i in live if done[i] + 1 == len(reqs[i])]
            steps.append({"step": s, "entries": [{"id": f"b{first_step}_{i}", "tokens": [reqs[i][done[i]]],
                                                  "want": [0]} for i in live],
                          "end": [f"b{first_step}_{i}" for i in ending]})
            expect[s] = torch.cat([refs[i][done[i]:done[i] + 1] for i in live])
            for i in live:
                done[i] += 1
            live = [i for i in live if done[i] < len(reqs[i])]
            s += 1
        return steps, expect, s

    s1, e1, nxt = batch_steps([0, 1, 2, 3], 0)
    s2, e2, _ = batch_steps([3, 2, 1], nxt)
    out = str(tmp_path / "batched")
    run_trace(folder, dtype, out, 64 + 128 + 64 + 192, s1 + s2)
    for s, r in {**e1, **e2}.items():
        assert near(read(out, s, V), r)
