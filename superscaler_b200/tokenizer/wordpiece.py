"""WordPiece tokenisation (the BERT scheme): clean-up and optional lower-casing / accent stripping, a split on
whitespace and punctuation (CJK characters stand alone), then a greedy longest-match-first split of every word into
vocabulary pieces, continuation pieces carrying the "##" prefix.
(reference: runtime/megatron/tokenizer/bert_tokenization.py)"""
from __future__ import annotations

import unicodedata
from typing import Dict, List


def load_vocab(path: str) -> Dict[str, int]:
    vocab: Dict[str, int] = {}
    with open(path, encoding="utf-8") as f:
        for line in f:
            tok = line.rstrip("\n")
            if tok and tok not in vocab:
                vocab[tok] = len(vocab)
    return vocab


def _is_punct(ch: str) -> bool:
    cp = ord(ch)
    if 33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126:
        return True
    return unicodedata.category(ch).startswith("P")


def _is_cjk(cp: int) -> bool:
    return (0x4E00 <= cp <= 0x9FFF or 0x3400 <= cp <= 0x4DBF or 0x20000 <= cp <= 0x2A6DF or 0x2A700 <= cp <= 0x2B73F
            or 0x2B740 <= cp <= 0x2B81F or 0x2B820 <= cp <= 0x2CEAF or 0xF900 <= cp <= 0xFAFF
            or 0x2F800 <= cp <= 0x2FA1F)


def basic_split(text: str, lower_case: bool = True) -> List[str]:
    cleaned = []
    for ch in text:
        cp = ord(ch)
        if cp == 0 or cp == 0xFFFD or (unicodedata.category(ch) in ("Cc", "Cf") and ch not in "\t\n\r"):
            continue
        if ch in " \t\n\r" or unicodedata.category(ch) == "Zs":
            cleaned.append(" ")
        elif _is_cjk(cp):
            cleaned.append(f" {ch} ")
        else:
            cleaned.append(ch)
    out: List[str] = []
    for word in "".join(cleaned).split():
        if lower_case:
            word = "".join(c for c in unicodedata.normalize("NFD", word.lower()) if unicodedata.category(c) != "Mn")
        cur = ""
        for ch in word:
            if _is_punct(ch):
                if cur:
                    out.append(cur)
                out.append(ch)
                cur = ""
            else:
                cur += ch
        if cur:
            out.append(cur)
    return out


class WordPieceEncoder:
    def __init__(self, vocab: Dict[str, int], lower_case: bool = True, unk: str = "[UNK]", max_word_chars: int = 200):
        self.vocab, self.lower_case, self.unk, self.max_word_chars = vocab, lower_case, unk, max_word_chars
        self.inverse = {i: s for s, i in vocab.items()}

    def pieces(self, word: str) -> List[str]:
        if len(word) > self.max_word_chars:
            return [self.unk]
        out, start = [], 0
        while start < len(word):
            end, found = len(word), None
            while end > start:
                cand = ("##" if start else "") + word[start:end]
                if cand in self.vocab:
                    found = cand
                    break
                end -= 1
            if found is None:
                return [self.unk]
            out.append(found)
            start = end
        return out

    def tokenize(self, text: str) -> List[str]:
        return [p for w in basic_split(text, self.lower_case) for p in self.pieces(w)]

    def encode(self, text: str) -> List[int]:
        return [self.vocab[p] for p in self.tokenize(text)]

    def decode(self, ids: List[int]) -> str:
        text = ""
        for i in ids:
            tok = self.inverse[int(i)]
            text += tok[2:] if tok.startswith("##") else ((" " if text else "") + tok)
        return text
