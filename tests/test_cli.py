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
    r = run("--model", "x", "--prompt", "hello")                  # no tokenizer.json in the folder
    assert r.returncode == 2 and "tokenizer not found" in r.stderr
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


@pytest.mark.gpu
def test_text_in_and_out_with_the_tokenizer(tmp_path):
    """--prompt with --tok: the ids are the tokenizer's, the completion is printed as ids and as text."""
    import shutil
    from brolm_b200.tokenizer import GemmaTokenizer
    folder = make_folder(tmp_path, "A", torch.float32)              # vocabulary of 256: the fixture's 43 ids fit
    fixture = os.path.join(ROOT, "tests", "golden", "tokenizer_fixture.json")
    shutil.copy(fixture, os.path.join(folder, "tokenizer.json"))    # found in the model folder without --tok
    config, weights = oracle_inputs(folder)
    tok = GemmaTokenizer.load(fixture)
    r = run("--model", folder, "--dtype", "float32", "--prompt", "hello the cat", "--max-new", "5", "--no-eos")
    assert r.returncode == 0, r.stderr
    lines = r.stdout.splitlines()
    ids = [config.get("bos_token_id", 2)] + tok.tokenize("hello the cat")
    assert list(map(int, lines[lines.index("--- prompt ---") + 1].split())) == ids
    got = list(map(int, lines[lines.index("--- completion ---") + 1].split()))
    assert got == plain.greedy(config, weights, ids, 5)
    assert lines[lines.index("--- text ---") + 1] == tok.decode(got)
    r = run("--model", folder, "--dtype", "float32", "--prompt", "a cat", "--chat", "--max-new", "2", "--no-eos")
    assert r.returncode == 0, r.stderr
    chat = list(map(int, r.stdout.splitlines()[r.stdout.splitlines().index("--- prompt ---") + 1].split()))
    assert chat[1] == tok.vocab["<start_of_turn>"] and tok.vocab["<end_of_turn>"] in chat
