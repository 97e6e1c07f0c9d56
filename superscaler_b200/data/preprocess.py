"""Turns text into the token corpus the training entry point reads (`runtime.pretrain --data-path <prefix>`).

    python -m superscaler_b200.data.preprocess --input corpus.jsonl [--json-key text] --output <prefix> \
        --tokenizer-type GPT2BPETokenizer --vocab-file vocab.json --merge-file merges.txt [--no-append-eod]
    python -m superscaler_b200.data.preprocess --input corpus.jsonl --output <prefix> --split-sentences \
        --tokenizer-type BertWordPieceLowerCase --vocab-file vocab.txt        # for BERT (and T5 span corruption)

Input: one document per line, either plain text or a JSON object with the text under --json-key.  Output:
`<prefix>.bin` (uint16 token ids, or `<prefix>.u32` when the vocabulary has more than 65536 entries) and
`<prefix>.npy` (int32 document lengths).  Every document ends with the tokenizer's end-of-document id unless
--no-append-eod is given (reference: the inherited Megatron preprocessing, runtime/megatron/data/test/).

With --split-sentences every document is cut into sentences (after ., ! or ? followed by white space, and at line
breaks inside the document text; the reference uses the nltk punkt splitter, which is not a dependency here), no
end-of-document id is added, and two more files describe the structure the sentence datasets need
(`data.sentences.SentenceCorpus`): `<prefix>.sent.npy` (int32 sentence lengths) and `<prefix>.docs.npy` (int64, for
document d the index of its first sentence; one more entry at the end = number of sentences).
"""
from __future__ import annotations

import argparse
import json
import re
from typing import Iterable, Iterator, List

import numpy as np

from ..tokenizer import build_tokenizer


def documents(path: str, json_key: str) -> Iterator[str]:
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.rstrip("\n")
            if not line.strip():
                continue
            if line.lstrip().startswith("{"):
                try:
                    yield json.loads(line)[json_key]
                    continue
                except (json.JSONDecodeError, KeyError):
                    pass
            yield line


def write_corpus(docs: Iterable[List[int]], prefix: str, vocab_size: int) -> int:
    """Writes the two files; returns the number of tokens."""
    wide = vocab_size > 65536
    dtype = np.uint32 if wide else np.uint16
    lengths, total = [], 0
    with open(prefix + (".u32" if wide else ".bin"), "wb") as out:
        for ids in docs:
            if not ids:
                continue
            np.asarray(ids, dtype=dtype).tofile(out)
            lengths.append(len(ids))
            total += len(ids)
    np.save(prefix + ".npy", np.asarray(lengths, dtype=np.int32))
    return total


_SENTENCE_END = re.compile(r"(?<=[.!?])\s+|\n+")


def split_sentences(text: str) -> List[str]:
    return [s.strip() for s in _SENTENCE_END.split(text) if s and s.strip()]


def write_sentence_corpus(docs: Iterable[List[List[int]]], prefix: str, vocab_size: int) -> int:
    """docs: for every document the token ids of its sentences.  Returns the number of tokens."""
    wide = vocab_size > 65536
    dtype = np.uint32 if wide else np.uint16
    sent_lengths, doc_starts, total = [], [0], 0
    with open(prefix + (".u32" if wide else ".bin"), "wb") as out:
        for sents in docs:
            sents = [s for s in sents if s]
            if not sents:
                continue
            for ids in sents:
                np.asarray(ids, dtype=dtype).tofile(out)
                sent_lengths.append(len(ids))
                total += len(ids)
            doc_starts.append(len(sent_lengths))
    np.save(prefix + ".sent.npy", np.asarray(sent_lengths, dtype=np.int32))
    np.save(prefix + ".docs.npy", np.asarray(doc_starts, dtype=np.int64))
    return total


def load_sentence_corpus(prefix: str):
    """The SentenceCorpus written by --split-sentences (tokens memory-mapped), or a sentence-split corpus in
    Megatron-LM's format (`<prefix>.idx`)."""
    import os

    from . import mmap_format
    from .sentences import SentenceCorpus
    if mmap_format.exists(prefix) and not os.path.exists(prefix + ".sent.npy"):
        return mmap_format.sentence_corpus(prefix)
    wide = os.path.exists(prefix + ".u32")
    tokens = np.memmap(prefix + (".u32" if wide else ".bin"), dtype=np.uint32 if wide else np.uint16, mode="r")
    return SentenceCorpus(tokens, np.load(prefix + ".sent.npy"), np.load(prefix + ".docs.npy"))


def write_megatron(a, tok) -> int:
    """The same corpus in Megatron-LM's format: items are sentences with --split-sentences, else documents (closed
    by the end-of-document id unless --no-append-eod)."""
    from . import mmap_format
    eod = None if a.no_append_eod else getattr(tok, "eod", getattr(tok, "sep", None))
    doc_idx = [0]

    def items():
        for text in documents(a.input, a.json_key):
            if a.split_sentences:
                sents = [s for s in (tok.tokenize(t) for t in split_sentences(text)) if s]
            else:
                ids = tok.tokenize(text)
                sents = [ids + [eod] if eod is not None else ids] if ids else []
            if not sents:
                continue
            yield from sents
            doc_idx.append(doc_idx[-1] + len(sents))

    dtype = np.uint16 if tok.vocab_size < 65500 else np.int32      # the reference's choice of element type
    return mmap_format.write(a.output, items(), doc_idx, dtype=dtype)     # doc_idx fills while the items are read


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True, help="prefix of the two output files")
    ap.add_argument("--json-key", default="text")
    ap.add_argument("--tokenizer-type", default="GPT2BPETokenizer")
    ap.add_argument("--vocab-file", required=True)
    ap.add_argument("--merge-file", default=None)
    ap.add_argument("--no-append-eod", action="store_true")
    ap.add_argument("--split-sentences", action="store_true")
    ap.add_argument("--output-format", choices=("native", "megatron"), default="native",
                    help="megatron: <prefix>.bin + <prefix>.idx as Megatron-LM's preprocessing writes them")
    a = ap.parse_args(argv)
    tok = build_tokenizer(a.tokenizer_type, a.vocab_file, a.merge_file)
    if a.output_format == "megatron":
        n = write_megatron(a, tok)
        print(f"wrote {a.output}.bin/.idx: {n} tokens, vocabulary {tok.vocab_size} (padded {tok.padded_vocab_size})")
        return
    if a.split_sentences:
        n = write_sentence_corpus(([tok.tokenize(s) for s in split_sentences(text)] for text in documents(a.input, a.json_key)),
                                  a.output, tok.vocab_size)
        print(f"wrote {a.output}: {n} tokens in sentences, vocabulary {tok.vocab_size} (padded {tok.padded_vocab_size})")
        return
    eod = None if a.no_append_eod else getattr(tok, "eod", getattr(tok, "sep", None))

    def encoded():
        for text in documents(a.input, a.json_key):
            ids = tok.tokenize(text)
            yield ids + [eod] if (eod is not None and ids) else ids

    n = write_corpus(encoded(), a.output, tok.vocab_size)
    print(f"wrote {a.output}: {n} tokens, vocabulary {tok.vocab_size} (padded {tok.padded_vocab_size})")


if __name__ == "__main__":
    main()
