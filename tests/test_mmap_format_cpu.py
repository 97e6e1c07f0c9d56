"""Megatron-LM's memory-mapped corpus format: round trip, the byte layout of the index, and use by the datasets."""
import json
import struct

import numpy as np
import pytest

from superscaler_b200.data import mmap_format
from superscaler_b200.data.indexed import GPTSampleDataset
from superscaler_b200.data.preprocess import load_sentence_corpus, main as preprocess_main


def test_index_layout_and_round_trip(tmp_path):
    prefix = str(tmp_path / "c")
    items = [[5, 6, 7], [8], [9, 10, 11, 12], [13, 14]]
    n = mmap_format.write(prefix, items, [0, 2, 4], dtype=np.uint16)
    assert n == 10
    raw = open(prefix + ".idx", "rb").read()
    assert raw[:9] == b"MMIDIDX\x00\x00"
    assert struct.unpack_from("<QBQQ", raw, 9) == (1, 8, 4, 3)
    at = 9 + 8 + 1 + 16
    assert np.frombuffer(raw, np.int32, 4, at).tolist() == [3, 1, 4, 2]
    assert np.frombuffer(raw, np.int64, 4, at + 16).tolist() == [0, 6, 8, 16]          # byte offsets of uint16 items
    assert np.frombuffer(raw, np.int64, 3, at + 16 + 32).tolist() == [0, 2, 4]
    assert len(raw) == at + 16 + 32 + 24
    elements, sizes, doc_idx = mmap_format.read(prefix)
    assert elements.dtype == np.uint16 and elements.tolist() == list(range(5, 15))
    assert sizes.tolist() == [3, 1, 4, 2] and doc_idx.tolist() == [0, 2, 4]
    s = mmap_format.sentence_corpus(prefix)
    assert [x.tolist() for x in s.sentences(2, 4)] == [[9, 10, 11, 12], [13, 14]]
    t = mmap_format.token_corpus(prefix)                 # sentences joined into their documents
    assert t.sizes.tolist() == [4, 6]


def test_int32_elements_and_bad_files(tmp_path):
    prefix = str(tmp_path / "w")
    mmap_format.write(prefix, [[70000, 1], [2]], [0, 1, 2], dtype=np.int32)
    elements, sizes, _ = mmap_format.read(prefix)
    assert elements.dtype == np.int32 and elements.tolist() == [70000, 1, 2] and sizes.tolist() == [2, 1]
    with open(prefix + ".bin", "ab") as f:
        f.write(b"\0\0\0\0")
    with pytest.raises(ValueError, match="adds up"):
        mmap_format.read(prefix)
    bad = str(tmp_path / "bad")
    open(bad + ".idx", "wb").write(b"TNTIDX\x00\x00" + b"\0" * 40)
    open(bad + ".bin", "wb").write(b"")
    with pytest.raises(ValueError, match="not a memory-mapped"):
        mmap_format.read(bad)


def _wordpiece_vocab(path):
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "the", "cat", "sat", "on", "mat", "dog", "ran", ".", "a"]
    path.write_text("\n".join(words) + "\n")


def test_preprocess_writes_a_corpus_the_datasets_read(tmp_path):
    vocab = tmp_path / "vocab.txt"
    _wordpiece_vocab(vocab)
    src = tmp_path / "in.jsonl"
    src.write_text("\n".join(json.dumps({"text": t}) for t in
                             ["the cat sat on the mat. a dog ran.", "a cat ran. the dog sat. the mat sat on a cat."]))
    prefix = str(tmp_path / "sent")
    preprocess_main(["--input", str(src), "--output", prefix, "--split-sentences", "--output-format", "megatron",
                     "--tokenizer-type", "BertWordPieceLowerCase", "--vocab-file", str(vocab)])
    c = load_sentence_corpus(prefix)                     # no .sent.npy beside it: read through the .idx file
    assert c.doc_starts.tolist() == [0, 2, 5]
    assert c.sizes.tolist() == [7, 4, 4, 4, 7]
    assert c.sentences(0, 1)[0].tolist() == [5, 6, 7, 8, 5, 9, 12]

    docs = str(tmp_path / "docs")
    preprocess_main(["--input", str(src), "--output", docs, "--output-format", "megatron",
                     "--tokenizer-type", "BertWordPieceLowerCase", "--vocab-file", str(vocab)])
    t = mmap_format.token_corpus(docs)
    assert t.sizes.tolist() == [12, 16]                  # 11 and 15 word pieces, each document closed by [SEP]
    assert t.tokens[11] == 3 and t.tokens[-1] == 3
    data = GPTSampleDataset(t, 4, num_samples=8, seed=1)
    assert len(data) >= 8 and data[0].shape == (5,)


def test_split_bounds_and_corpus_slices():
    from superscaler_b200.data.indexed import TokenCorpus, split_bounds
    from superscaler_b200.data.sentences import SentenceCorpus
    assert split_bounds("949,50,1", 1000) == [0, 949, 999, 1000]
    assert split_bounds("98/2", 50) == [0, 49, 50, 50]
    assert split_bounds("1", 7) == [0, 7, 7, 7]
    b = split_bounds("1,1,1", 10)                        # 3 + 3 + 3 = 9: the missing document moves every boundary up
    assert b == [0, 4, 7, 10]
    t = TokenCorpus(np.arange(10), [3, 2, 5])
    part = t.slice_docs(1, 3)
    assert part.tokens.tolist() == list(range(3, 10)) and part.sizes.tolist() == [2, 5]
    s = SentenceCorpus(np.arange(12), [2, 3, 1, 4, 2], [0, 2, 3, 5], title_lengths=[1, 2, 3])
    part = s.slice_docs(1, 3)
    assert part.tokens.tolist() == list(range(5, 12)) and part.sizes.tolist() == [1, 4, 2]
    assert part.doc_starts.tolist() == [0, 1, 3] and part.title_sizes.tolist() == [2, 3]
