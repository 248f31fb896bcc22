"""What bench.py answers without a GPU: more than one GPU is refused with one
line and exit code 2, the reference arm says in one JSON line why it cannot
run, and the count of a step's floating-point operations is that of the
layer sizes."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          cwd=ROOT, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = run("--gpus", "2")
    assert p.returncode == 2
    lines = [ln for ln in (p.stdout + p.stderr).splitlines() if ln.strip()]
    assert len(lines) == 1 and "one-GPU" in lines[0]


def test_reference_arm_is_unavailable_and_says_why():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    d = json.loads(p.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_prefill_flops_follow_the_layer_sizes():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    import brolm_b200 as bb
    cfg = bb.Gemma2Config()                    # the 2B defaults
    T, L = 2048, cfg.num_hidden_layers
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    products = 2.0 * T * (cfg.hidden_size * (q + 2 * kv) + q * cfg.hidden_size + 3 * cfg.hidden_size * cfg.intermediate_size)
    got = bench.prefill_flops(cfg, L, T)
    # the products of the layers are most of it; attention and the last token's output matrix come on top
    assert L * products <= got <= 1.25 * L * products
