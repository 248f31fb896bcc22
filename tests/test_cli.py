import os
import subprocess
import sys

import pytest
import torch

from tests.helpers import make_folder, oracle_inputs
from tests.plain import gemma2_plain as plain

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
TOOL = os.path.join(ROOT, "bin", "run_gemma2")


def run(*args):
    return subprocess.run([sys.executable, TOOL, *args], capture_output=True, text=True, timeout=600)


def test_arguments_are_checked_before_anything_is_loaded():
    assert run("--model", "x", "--prompt", "hello").returncode == 2
    assert run("--model", "x").returncode == 2                      # no ids
    assert run("--ids", "1,2").returncode == 2                      # neither --model nor --random
    r = run("--model", "/nonexistent", "--ids", "1,2", "--device", "cpu")
    assert r.returncode == 1 and "fatal" in r.stderr


@pytest.mark.gpu
def test_greedy_from_the_command_line_matches_the_oracle(tmp_path):
    folder = make_folder(tmp_path, "A", torch.float32)
    config, weights = oracle_inputs(folder)
    r = run("--model", folder, "--dtype", "float32", "--ids", "5,17,3,99", "--ids", "200 7", "--max-new", "6",
            "--no-eos")
    assert r.returncode == 0, r.stderr
    lines = r.stdout.splitlines()
    got = [list(map(int, lines[i + 1].split())) for i, l in enumerate(lines) if l == "--- completion ---"]
    bos = config.get("bos_token_id", 2)
    assert got == [plain.greedy(config, weights, [bos, 5, 17, 3, 99], 6), plain.greedy(config, weights, [bos, 200, 7], 6)]
