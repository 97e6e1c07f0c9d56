"""Turns text into the token corpus the GPT entry point reads (`runtime.pretrain --data-path <prefix>`).

    python -m superscaler_b200.data.preprocess --input corpus.jsonl [--json-key text] --output <prefix> \
        --tokenizer-type GPT2BPETokenizer --vocab-file vocab.json --merge-file merges.txt [--no-append-eod]

Input: one document per line, either plain text or a JSON object with the text under --json-key.  Output:
`<prefix>.bin` (uint16 token ids, or `<prefix>.u32` when the vocabulary has more than 65536 entries) and
`<prefix>.npy` (int32 document lengths).  Every document ends with the tokenizer's end-of-document id unless
--no-append-eod is given (reference: the inherited Megatron preprocessing, runtime/megatron/data/test/).
"""
from __future__ import annotations

import argparse
import json
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


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True, help="prefix of the two output files")
    ap.add_argument("--json-key", default="text")
    ap.add_argument("--tokenizer-type", default="GPT2BPETokenizer")
    ap.add_argument("--vocab-file", required=True)
    ap.add_argument("--merge-file", default=None)
    ap.add_argument("--no-append-eod", action="store_true")
    a = ap.parse_args(argv)
    tok = build_tokenizer(a.tokenizer_type, a.vocab_file, a.merge_file)
    eod = None if a.no_append_eod else getattr(tok, "eod", getattr(tok, "sep", None))

    def encoded():
        for text in documents(a.input, a.json_key):
            ids = tok.tokenize(text)
            yield ids + [eod] if (eod is not None and ids) else ids

    n = write_corpus(encoded(), a.output, tok.vocab_size)
    print(f"wrote {a.output}: {n} tokens, vocabulary {tok.vocab_size} (padded {tok.padded_vocab_size})")


if __name__ == "__main__":
    main()
