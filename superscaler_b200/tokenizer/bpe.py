"""Byte-level BPE (the GPT-2 scheme): text is split by a regular expression into word-like pieces, every piece is
turned into a sequence of printable stand-ins for its UTF-8 bytes, and adjacent symbols are merged greedily in the
priority order of the merge table.  (reference: runtime/megatron/tokenizer/gpt2_tokenization.py)"""
from __future__ import annotations

import json
from functools import lru_cache
from typing import Dict, List, Tuple

import regex

_SPLIT = regex.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+")


@lru_cache(maxsize=1)
def byte_symbols() -> Dict[int, str]:
    """byte value -> one printable unicode character; printable latin-1 bytes map to themselves, the rest to
    code points from 256 upwards, so that no symbol is whitespace or a control character."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class BytePairEncoder:
    def __init__(self, vocab: Dict[str, int], merges: List[Tuple[str, str]]):
        self.vocab = vocab
        self.inverse = {i: s for s, i in vocab.items()}
        self.rank = {pair: i for i, pair in enumerate(merges)}
        self.to_symbol = byte_symbols()
        self.to_byte = {s: b for b, s in self.to_symbol.items()}
        self._cache: Dict[str, List[str]] = {}

    @classmethod
    def from_files(cls, vocab_file: str, merge_file: str) -> "BytePairEncoder":
        with open(vocab_file, encoding="utf-8") as f:
            vocab = json.load(f)
        merges = []
        with open(merge_file, encoding="utf-8") as f:
            for line in f:
                line = line.rstrip("\n")
                if not line or line.startswith("#version"):
                    continue
                a, b = line.split(" ")
                merges.append((a, b))
        return cls(vocab, merges)

    def _merge_word(self, word: str) -> List[str]:
        if word in self._cache:
            return self._cache[word]
        parts = list(word)
        while len(parts) > 1:
            best, best_rank = None, None
            for i in range(len(parts) - 1):
                r = self.rank.get((parts[i], parts[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = (parts[i], parts[i + 1]), r
            if best is None:
                break
            merged, i = [], 0
            while i < len(parts):
                if i + 1 < len(parts) and (parts[i], parts[i + 1]) == best:
                    merged.append(parts[i] + parts[i + 1])
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        self._cache[word] = parts
        return parts

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for piece in _SPLIT.findall(text):
            word = "".join(self.to_symbol[b] for b in piece.encode("utf-8"))
            ids.extend(self.vocab[s] for s in self._merge_word(word))
        return ids

    def decode(self, ids: List[int]) -> str:
        symbols = "".join(self.inverse[int(i)] for i in ids)
        return bytes(self.to_byte[s] for s in symbols).decode("utf-8", errors="replace")
