"""The Gemma / Gemma 2 tokenizer: SentencePiece-style BPE read from a HuggingFace ``tokenizer.json``.

What it does is what wlejon/brolm's ``gemma::Tokenizer`` does (include/brolm/gemma_tokenizer.h:5-24,
src/gemma_tokenizer.cpp:19-154, src/detail/spm_bpe.cpp:81-149):

* added tokens (``<bos>``, ``<start_of_turn>``, ...) are matched verbatim in the text, the longest one
  at a position wins, and become their single id (include/brolm/detail/byte_level_bpe.h:164-194);
* the text between them has every ASCII space replaced by U+2581 and **no** space is put in front
  (Gemma's "no prefix space"); it is cut into words that each begin at a U+2581, so that no merge
  reaches across a word;
* a word starts as its characters; a character that is no piece of the vocabulary becomes one
  ``<0xNN>`` piece per UTF-8 byte (byte fallback); then the adjacent pair with the lowest merge rank
  (the leftmost of equals) is joined until no listed pair is left; pieces that the vocabulary does not
  have become ``<unk>``;
* decoding joins the pieces' bytes, turns ``<0xNN>`` pieces back into their byte and U+2581 into a
  space; ids outside the vocabulary are skipped.

The test ``tests/test_tokenizer.py`` compares it with the output of brolm's own tokenizer, compiled
here on the CPU, on a small vocabulary (``tests/golden/tokenizer_cases.*``).
"""
from __future__ import annotations

import json
import re
from typing import Iterable, Optional

METASPACE = "▁"
_BYTE_PIECE = re.compile(r"^<0[xX]([0-9a-fA-F]{2})>$")


class TokenizerError(ValueError):
    pass


class GemmaTokenizer:
    def __init__(self, vocab: dict, merges: list, added: list, byte_fallback: bool = True, fuse_unk: bool = False):
        self.vocab: dict[str, int] = dict(vocab)
        self.byte_fallback, self.fuse_unk = bool(byte_fallback), bool(fuse_unk)
        self.ranks: dict[tuple, int] = {}
        for rank, (left, right) in enumerate(merges):
            self.ranks.setdefault((left, right), rank)           # the first listing of a pair keeps its rank
        self.pieces: dict[int, str] = {i: p for p, i in self.vocab.items() if i >= 0}
        self.specials: dict[str, int] = {}
        named = dict(self.vocab)
        for content, token_id in added:
            if not content:
                continue
            self.specials[content] = token_id
            if content not in self.vocab and token_id >= 0:
                self.pieces[token_id] = content                  # decodable, never produced by a merge
            named[content] = token_id
        # longest first, so that the first match at a position is the longest one
        self._specials_by_length = sorted(self.specials, key=len, reverse=True)
        self._special_starts = {s[0] for s in self.specials}
        self.pad_id = named.get("<pad>", 0)
        self.eos_id = named.get("<eos>", 1)
        self.bos_id = named.get("<bos>", 2)
        self.unk_id = named.get("<unk>", 3)

    # loading ----------------------------------------------------------------
    @classmethod
    def load(cls, path: str) -> "GemmaTokenizer":
        """Read a HuggingFace tokenizer.json (its ``model`` must be a BPE with ``vocab`` and ``merges``)."""
        try:
            with open(path, "r", encoding="utf-8") as fh:
                root = json.load(fh)
        except OSError:
            raise TokenizerError(f"GemmaTokenizer: cannot open '{path}'") from None
        except json.JSONDecodeError as e:
            raise TokenizerError(f"GemmaTokenizer: json parse: {e}") from None
        model = root.get("model") if isinstance(root, dict) else None
        if not isinstance(model, dict):
            raise TokenizerError("GemmaTokenizer: tokenizer.json has no 'model' object")
        if model.get("type", "") != "BPE":
            raise TokenizerError(f"GemmaTokenizer: expected a BPE model, got '{model.get('type', '')}'")
        vocab = model.get("vocab")
        if not isinstance(vocab, dict) or not vocab:
            raise TokenizerError("GemmaTokenizer: model has no BPE 'vocab' object")
        if not isinstance(model.get("merges"), list):
            raise TokenizerError("GemmaTokenizer: model has no 'merges' array")
        merges = []
        for entry in model["merges"]:
            if isinstance(entry, list) and len(entry) >= 2:
                merges.append((str(entry[0]), str(entry[1])))
            elif isinstance(entry, str) and " " in entry:
                left, right = entry.split(" ", 1)
                merges.append((left, right))
            else:
                merges.append((None, None))                      # keeps the ranks of the entries after it
        added = []
        for entry in root.get("added_tokens") or []:
            if isinstance(entry, dict) and isinstance(entry.get("content"), str) and "id" in entry:
                added.append((entry["content"], int(entry["id"])))
        byte_fallback = model.get("byte_fallback")
        fuse_unk = model.get("fuse_unk")
        return cls({p: int(i) for p, i in vocab.items()}, merges, added,
                   True if byte_fallback is None else bool(byte_fallback), bool(fuse_unk))

    @property
    def vocab_count(self) -> int:
        return len(self.vocab)

    # text -> ids --------------------------------------------------------------
    def _word(self, word: str, out: list) -> None:
        symbols: list[str] = []
        for ch in word:
            if ch in self.vocab or not self.byte_fallback:
                symbols.append(ch)
            else:
                symbols.extend(f"<0x{b:02X}>" for b in ch.encode("utf-8"))
        ranks = self.ranks
        while len(symbols) > 1:
            best, at = None, -1
            for j in range(len(symbols) - 1):
                r = ranks.get((symbols[j], symbols[j + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, j
            if best is None:
                break
            symbols[at:at + 2] = [symbols[at] + symbols[at + 1]]
        for s in symbols:
            token_id = self.vocab.get(s)
            if token_id is not None:
                out.append(token_id)
            elif not self.fuse_unk or not out or out[-1] != self.unk_id:
                out.append(self.unk_id)

    def _span(self, text: str, out: list) -> None:
        """Plain text (no added tokens in it): metaspace, words, merges."""
        s = text.replace(" ", METASPACE)
        start = 0
        while start < len(s):
            nxt = s.find(METASPACE, start + 1)
            if nxt < 0:
                nxt = len(s)
            self._word(s[start:nxt], out)
            start = nxt

    def tokenize(self, text: str) -> list[int]:
        """Ids of ``text`` without ``<bos>`` / ``<eos>``; added tokens in the text become their ids."""
        out: list[int] = []
        i = span_start = 0
        n = len(text)
        while i < n:
            hit = None
            if text[i] in self._special_starts:
                for s in self._specials_by_length:
                    if text.startswith(s, i):
                        hit = s
                        break
            if hit is None:
                i += 1
                continue
            if i > span_start:
                self._span(text[span_start:i], out)
            out.append(self.specials[hit])
            i += len(hit)
            span_start = i
        if n > span_start:
            self._span(text[span_start:], out)
        return out

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = False) -> list[int]:
        """``[<bos>] + tokenize(text) + [<eos>]`` (defaults as brolm's: with ``<bos>``, without ``<eos>``)."""
        return ([self.bos_id] if add_bos else []) + self.tokenize(text) + ([self.eos_id] if add_eos else [])

    # ids -> text --------------------------------------------------------------
    def decode_bytes(self, ids: Iterable[int], skip: Optional[set] = None) -> bytes:
        raw = bytearray()
        for token_id in ids:
            piece = self.pieces.get(int(token_id))
            if piece is None or (skip and int(token_id) in skip):
                continue
            m = _BYTE_PIECE.match(piece)
            if m:
                raw.append(int(m.group(1), 16))
            else:
                raw += piece.encode("utf-8")
        return bytes(raw).replace(METASPACE.encode("utf-8"), b" ")

    def decode(self, ids: Iterable[int], skip: Optional[set] = None) -> str:
        """The text of ``ids``; bytes that are no valid UTF-8 (half of a character) show as U+FFFD."""
        return self.decode_bytes(ids, skip).decode("utf-8", errors="replace")
