"""The tokenizer against wlejon/brolm's own, compiled on the CPU: ``tests/golden/tokenizer_cases.expected`` is
the output of ``tests/golden/tokenizer_cases.cpp`` (brolm's src/gemma_tokenizer.cpp, src/detail/spm_bpe.cpp and
src/detail/byte_level_bpe.cpp, which build without brotensor) for the texts in ``tokenizer_cases.txt`` and the
small ``tokenizer_fixture.json``.  With a checkout of brolm at ``$BROLM_REFERENCE`` and g++ at hand the
program is built and run again first, so the committed output is known to be still the reference's."""
import json
import os
import shutil
import subprocess

import pytest

from brolm_b200.tokenizer import GemmaTokenizer, TokenizerError

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FIXTURE = os.path.join(HERE, "tokenizer_fixture.json")


def golden(tmp_path):
    expected = open(os.path.join(HERE, "tokenizer_cases.expected")).read()
    ref = os.environ.get("BROLM_REFERENCE", "")
    sources = [os.path.join(ref, "src", f) for f in ("gemma_tokenizer.cpp", "detail/spm_bpe.cpp", "detail/byte_level_bpe.cpp")]
    if shutil.which("g++") and all(os.path.exists(s) for s in sources):
        exe = str(tmp_path / "tokenizer_cases")
        subprocess.check_call(["g++", "-std=c++20", "-O1", "-I", os.path.join(ref, "include"),
                               os.path.join(HERE, "tokenizer_cases.cpp"), *sources, "-o", exe])
        again = subprocess.check_output([exe, FIXTURE, os.path.join(HERE, "tokenizer_cases.txt")], text=True)
        assert again == expected
    return expected.splitlines()


def test_ids_and_text_equal_the_references(tmp_path):
    lines = golden(tmp_path)
    tok = GemmaTokenizer.load(FIXTURE)
    head = lines[0].split()
    assert [tok.pad_id, tok.eos_id, tok.bos_id, tok.unk_id, tok.vocab_count] == [int(head[i]) for i in (2, 4, 6, 8, 10)]
    texts = [bytes.fromhex(l.strip()).decode("utf-8") for l in open(os.path.join(HERE, "tokenizer_cases.txt"))]
    assert len(lines) == 1 + 3 * len(texts)
    for n, text in enumerate(texts):
        want_tok = [int(v) for v in lines[1 + 3 * n].split()[1:]]
        want_enc = [int(v) for v in lines[2 + 3 * n].split()[1:]]
        want_dec = bytes.fromhex(lines[3 + 3 * n].split(" ", 1)[1].strip()) if len(lines[3 + 3 * n].split()) > 1 else b""
        assert tok.tokenize(text) == want_tok, repr(text)
        assert tok.encode(text, add_bos=True, add_eos=True) == want_enc, repr(text)
        assert tok.decode_bytes(want_tok) == want_dec, repr(text)


def test_framing_round_trip_and_errors(tmp_path):
    tok = GemmaTokenizer.load(FIXTURE)
    assert tok.encode("a cat") == [tok.bos_id] + tok.tokenize("a cat") and tok.encode("a cat", add_bos=False) == tok.tokenize("a cat")
    for text in ("a cat", " cat", "hello the cat", "caté at", "€"):
        assert tok.decode(tok.tokenize(text)) == text
    assert tok.decode([10 ** 6, -5]) == ""                      # ids outside the vocabulary are skipped
    assert tok.decode([tok.vocab["<0xC3>"]]) == "�"        # half a character
    with pytest.raises(TokenizerError, match="cannot open"):
        GemmaTokenizer.load(str(tmp_path / "missing.json"))
    for doc, what in (("{", "json parse"), ("{}", "no 'model'"), ('{"model": {"type": "Unigram"}}', "expected a BPE"),
                      ('{"model": {"type": "BPE", "vocab": {"a": 0}}}', "no 'merges'")):
        p = tmp_path / "t.json"
        p.write_text(doc)
        with pytest.raises(TokenizerError, match=what):
            GemmaTokenizer.load(str(p))
    # merges given as pairs, and the fused <unk>
    doc = json.load(open(FIXTURE))
    doc["model"]["merges"] = [m.split(" ", 1) for m in doc["model"]["merges"]]
    doc["model"]["byte_fallback"] = False
    doc["model"]["fuse_unk"] = True
    p = tmp_path / "pairs.json"
    p.write_text(json.dumps(doc, ensure_ascii=False))
    fused = GemmaTokenizer.load(str(p))
    assert fused.tokenize("a cat") == tok.tokenize("a cat")
    assert fused.tokenize("xyz") == [fused.unk_id] and tok.tokenize("xyz") == [tok.unk_id] * 3
