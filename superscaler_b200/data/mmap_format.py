"""Reads and writes the memory-mapped corpus format of Megatron-LM (`<prefix>.bin` + `<prefix>.idx`), so a corpus
preprocessed for the reference trains here without being converted, and a corpus written here loads there.

On-disk layout of `<prefix>.idx` (reference: MMapIndexedDataset.Index, runtime/megatron/data/indexed_dataset.py:335-420;
all integers little-endian):

    9 bytes   magic  "MMIDIDX\\0\\0"
    uint64    version (1)
    uint8     element type of the .bin file: 1 uint8, 2 int8, 3 int16, 4 int32, 5 int64, 6 float32, 7 float64, 8 uint16
    uint64    n  = number of items (sentences when the corpus was split into sentences, else documents)
    uint64    d  = number of entries of the document index
    int32[n]  item lengths, in elements
    int64[n]  byte offset of every item in the .bin file
    int64[d]  document index: item number at which every document starts, closed by n

`<prefix>.bin` is the items' elements back to back.  `read` hands out views of memory maps (nothing is loaded);
`token_corpus` / `sentence_corpus` wrap them as the two corpus classes the datasets here are built on.
"""
from __future__ import annotations

import os
import struct
from typing import Iterable, Sequence, Tuple

import numpy as np

MAGIC = b"MMIDIDX\x00\x00"
DTYPE_OF_CODE = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64,
                 8: np.uint16}
CODE_OF_DTYPE = {np.dtype(v): k for k, v in DTYPE_OF_CODE.items()}
_HEADER = struct.Struct("<9sQBQQ")


def exists(prefix: str) -> bool:
    return os.path.exists(prefix + ".idx") and os.path.exists(prefix + ".bin")


def read(prefix: str) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(elements, item lengths int32, document index int64) of the corpus at `prefix`; raises ValueError when the
    files are not of this format or do not fit each other."""
    path = prefix + ".idx"
    with open(path, "rb") as f:
        head = f.read(_HEADER.size)
    if len(head) < _HEADER.size:
        raise ValueError(f"{path}: too short for an index header")
    magic, version, code, n, d = _HEADER.unpack(head)
    if magic != MAGIC:
        raise ValueError(f"{path}: not a memory-mapped corpus index (magic {magic!r})")
    if version != 1 or code not in DTYPE_OF_CODE:
        raise ValueError(f"{path}: version {version}, element type code {code} not understood")
    need = _HEADER.size + 4 * n + 8 * n + 8 * d
    if os.path.getsize(path) < need:
        raise ValueError(f"{path}: {os.path.getsize(path)} bytes, the header promises {need}")
    raw = np.memmap(path, dtype=np.uint8, mode="r")
    at = _HEADER.size
    sizes = np.frombuffer(raw, dtype=np.int32, count=n, offset=at)
    pointers = np.frombuffer(raw, dtype=np.int64, count=n, offset=at + 4 * n)
    doc_idx = np.frombuffer(raw, dtype=np.int64, count=d, offset=at + 12 * n)
    dtype = np.dtype(DTYPE_OF_CODE[code])
    total = int(sizes.sum(dtype=np.int64))
    elements = np.memmap(prefix + ".bin", dtype=dtype, mode="r") if total else np.zeros(0, dtype)
    if len(elements) != total:
        raise ValueError(f"{prefix}.bin holds {len(elements)} elements, the index adds up to {total}")
    if n and (pointers[0] != 0 or int(pointers[-1]) != (total - int(sizes[-1])) * dtype.itemsize):
        raise ValueError(f"{path}: items are not stored back to back")
    return elements, sizes, doc_idx


def write(prefix: str, items: Iterable[Sequence[int]], doc_idx: Sequence[int], dtype=np.uint16) -> int:
    """Writes `<prefix>.bin` and `<prefix>.idx`; `doc_idx` as in the layout above (it is read only after `items`
    is exhausted, so a generator may fill it as it goes).  Returns the number of elements."""
    dtype = np.dtype(dtype)
    sizes = []
    with open(prefix + ".bin", "wb") as out:
        for ids in items:
            np.asarray(ids, dtype=dtype).tofile(out)
            sizes.append(len(ids))
    sizes = np.asarray(sizes, dtype=np.int32)
    doc_idx = np.asarray(doc_idx, dtype=np.int64)
    assert len(doc_idx) == 0 or (doc_idx[0] == 0 and doc_idx[-1] == len(sizes)), "document index must span the items"
    pointers = np.zeros(len(sizes), dtype=np.int64)
    if len(sizes) > 1:
        np.cumsum(sizes[:-1].astype(np.int64) * dtype.itemsize, out=pointers[1:])
    with open(prefix + ".idx", "wb") as out:
        out.write(_HEADER.pack(MAGIC, 1, CODE_OF_DTYPE[dtype], len(sizes), len(doc_idx)))
        out.write(sizes.tobytes())
        out.write(pointers.tobytes())
        out.write(doc_idx.tobytes())
    return int(sizes.sum(dtype=np.int64))


def token_corpus(prefix: str):
    """A corpus whose items are whole documents (the reference's GPT preprocessing) as a `TokenCorpus`.  A corpus
    split into sentences is accepted as well: its sentences are joined into documents by the document index."""
    from .indexed import TokenCorpus
    elements, sizes, doc_idx = read(prefix)
    if len(doc_idx) == len(sizes) + 1 or len(doc_idx) == 0:
        return TokenCorpus(elements, sizes)
    ends = np.concatenate([[0], np.cumsum(sizes, dtype=np.int64)])
    lengths = ends[doc_idx[1:]] - ends[doc_idx[:-1]]
    return TokenCorpus(elements, lengths[lengths > 0])


def sentence_corpus(prefix: str):
    """A corpus preprocessed with sentence splitting as a `SentenceCorpus` (items = sentences)."""
    from .sentences import SentenceCorpus
    elements, sizes, doc_idx = read(prefix)
    if len(doc_idx) == 0:
        doc_idx = np.arange(len(sizes) + 1, dtype=np.int64)
    return SentenceCorpus(elements, sizes, doc_idx)
