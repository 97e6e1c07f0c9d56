"""Tokenizer front ends and the vocabulary padding rule.

`padded_vocab_size`: the embedding table is padded so that every tensor-parallel shard has a multiple of 128 rows
(reference: _vocab_size_with_padding, runtime/megatron/tokenizer/tokenizer.py:54-71; GPT-2's 50257 becomes 50304
at tp = 1).  `build_tokenizer(kind, ...)` returns a GPT-2 BPE or a BERT WordPiece tokenizer with the special ids
the datasets need (eod / cls / sep / pad / mask / bos / eos and the `<extra_id_i>` sentinels of T5)."""
from __future__ import annotations

from typing import Dict, List, Optional

from .bpe import BytePairEncoder
from .wordpiece import WordPieceEncoder, load_vocab


def padded_vocab_size(vocab_size: int, tp: int = 1, divisible_by: int = 128) -> int:
    multiple = divisible_by * tp
    return (vocab_size + multiple - 1) // multiple * multiple


class GPT2BPETokenizer:
    def __init__(self, vocab_file: str, merge_file: str):
        self.bpe = BytePairEncoder.from_files(vocab_file, merge_file)
        self.eod = self.bpe.vocab["<|endoftext|>"]

    @property
    def vocab_size(self) -> int:
        return len(self.bpe.vocab)

    @property
    def vocab(self) -> Dict[str, int]:
        return self.bpe.vocab

    def tokenize(self, text: str) -> List[int]:
        return self.bpe.encode(text)

    def detokenize(self, ids: List[int]) -> str:
        return self.bpe.decode(ids)


class BertWordPieceTokenizer:
    def __init__(self, vocab_file: str, lower_case: bool = True, vocab_extra_ids: int = 0):
        vocab = load_vocab(vocab_file)
        self.wp = WordPieceEncoder(vocab, lower_case)
        self.cls, self.sep, self.pad, self.mask = (vocab[t] for t in ("[CLS]", "[SEP]", "[PAD]", "[MASK]"))
        self.bos = self._add("[BOS]")
        self.eos = self._add("[EOS]")
        self.sentinels = [self._add(f"<extra_id_{i}>") for i in range(vocab_extra_ids)]

    def _add(self, token: str) -> int:
        v = self.wp.vocab
        if token not in v:
            v[token] = len(v)
            self.wp.inverse[v[token]] = token
        return v[token]

    @property
    def vocab_size(self) -> int:
        return len(self.wp.vocab)

    @property
    def vocab(self) -> Dict[str, int]:
        return self.wp.vocab

    def tokenize(self, text: str) -> List[int]:
        return self.wp.encode(text)

    def detokenize(self, ids: List[int]) -> str:
        skip = {self.cls, self.sep, self.pad}
        return self.wp.decode([i for i in ids if int(i) not in skip])

    def special_tokens(self):
        """The ids in the form the sentence datasets take."""
        from ..data.sentences import SpecialTokens
        return SpecialTokens(cls=self.cls, sep=self.sep, mask=self.mask, pad=self.pad, bos=self.bos, eos=self.eos,
                             sentinels=tuple(self.sentinels))


def build_tokenizer(kind: str, vocab_file: str, merge_file: Optional[str] = None, vocab_extra_ids: int = 0,
                    tp: int = 1, divisible_by: int = 128):
    """kind: GPT2BPETokenizer | BertWordPieceLowerCase | BertWordPieceCase.  The returned object also carries
    `padded_vocab_size` for the model's embedding table."""
    if kind == "GPT2BPETokenizer":
        assert merge_file is not None, "the BPE tokenizer needs a merge table"
        tok = GPT2BPETokenizer(vocab_file, merge_file)
    elif kind in ("BertWordPieceLowerCase", "BertWordPieceCase"):
        tok = BertWordPieceTokenizer(vocab_file, kind == "BertWordPieceLowerCase", vocab_extra_ids)
    else:
        raise NotImplementedError(f"{kind} tokenizer is not implemented")
    tok.padded_vocab_size = padded_vocab_size(tok.vocab_size, tp, divisible_by)
    return tok
