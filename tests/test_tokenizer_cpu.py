"""Tokenizers on small hand-made vocabularies (reference: runtime/megatron/tokenizer/)."""
import json

import pytest

from superscaler_b200.tokenizer import build_tokenizer, padded_vocab_size
from superscaler_b200.tokenizer.bpe import byte_symbols


def test_vocab_padding_rule():
    assert padded_vocab_size(50257) == 50304            # GPT-2 at tp = 1
    assert padded_vocab_size(50257, tp=8) == 51200
    assert padded_vocab_size(30522, tp=2) == 30720
    assert padded_vocab_size(51200, tp=8) == 51200


def _bpe_files(tmp_path):
    sym = byte_symbols()
    space = sym[ord(" ")]
    merges = [("l", "o"), ("lo", "w"), ("e", "r"), (space, "low"), ("n", "e"), ("ne", "w"), (space, "new")]
    vocab = {}
    for s in list(sym.values()) + [a + b for a, b in merges] + ["<|endoftext|>"]:
        vocab.setdefault(s, len(vocab))
    vf, mf = tmp_path / "vocab.json", tmp_path / "merges.txt"
    vf.write_text(json.dumps(vocab), encoding="utf-8")
    mf.write_text("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges) + "\n", encoding="utf-8")
    return str(vf), str(mf), vocab, space


def test_gpt2_bpe_merges_in_priority_order_and_round_trips(tmp_path):
    vf, mf, vocab, space = _bpe_files(tmp_path)
    tok = build_tokenizer("GPT2BPETokenizer", vf, mf)
    assert tok.vocab_size == len(vocab) and tok.padded_vocab_size % 128 == 0 and tok.eod == vocab["<|endoftext|>"]
    ids = tok.tokenize("low lower newer")
    inv = {i: s for s, i in vocab.items()}
    assert [inv[i] for i in ids] == ["low", space + "low", "er", space + "new", "er"]
    for text in ("low lower newer", "Hello, wörld! 123\n\ttabs  and  spaces ", "日本語 ok"):
        assert tok.detokenize(tok.tokenize(text)) == text


def test_byte_symbols_are_printable_and_unique():
    sym = byte_symbols()
    assert len(sym) == 256 and len(set(sym.values())) == 256
    assert all(not s.isspace() and s.isprintable() for s in sym.values())


def _wp_vocab(tmp_path):
    toks = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "the", "un", "##aff", "##able", "##s", "run", "##ning", ",",
            ".", "cafe", "中", "文", "a"]
    p = tmp_path / "vocab.txt"
    p.write_text("\n".join(toks) + "\n", encoding="utf-8")
    return str(p), toks


def test_wordpiece_longest_match_and_specials(tmp_path):
    path, toks = _wp_vocab(tmp_path)
    tok = build_tokenizer("BertWordPieceLowerCase", path, vocab_extra_ids=3)
    assert (tok.pad, tok.cls, tok.sep, tok.mask) == (0, 2, 3, 4)
    assert tok.vocab_size == len(toks) + 2 + 3 and len(tok.sentinels) == 3 and tok.bos != tok.eos
    assert tok.wp.tokenize("The unaffable runs, Café 中文.") == \
        ["the", "un", "##aff", "##able", "run", "##s", ",", "cafe", "中", "文", "."]
    assert tok.wp.tokenize("xyzzy running") == ["[UNK]", "run", "##ning"]
    ids = tok.tokenize("the unaffable")
    assert tok.detokenize([tok.cls] + ids + [tok.sep]) == "the unaffable"
    cased = build_tokenizer("BertWordPieceCase", path)
    assert cased.wp.tokenize("The a") == ["[UNK]", "a"]
    sp = tok.special_tokens()
    assert sp.sentinels == tuple(tok.sentinels) and sp.bos == tok.bos


def test_unknown_tokenizer_kind():
    with pytest.raises(NotImplementedError):
        build_tokenizer("SentencePiece", "x")


def test_preprocess_writes_a_corpus_the_dataset_reads(tmp_path, capsys):
    import numpy as np
    from superscaler_b200.data import preprocess
    from superscaler_b200.data.indexed import GPTSampleDataset, TokenCorpus
    vf, mf, vocab, space = _bpe_files(tmp_path)
    src = tmp_path / "docs.jsonl"
    src.write_text('{"text": "low lower newer"}\n\nnewer low\n{"text": "lower"}\n', encoding="utf-8")
    preprocess.main(["--input", str(src), "--output", str(tmp_path / "c"), "--vocab-file", vf, "--merge-file", mf])
    assert "tokens" in capsys.readouterr().out
    tok = build_tokenizer("GPT2BPETokenizer", vf, mf)
    lengths = np.load(tmp_path / "c.npy")
    tokens = np.fromfile(tmp_path / "c.bin", dtype=np.uint16)
    want = [tok.tokenize(t) + [tok.eod] for t in ("low lower newer", "newer low", "lower")]
    assert lengths.tolist() == [len(w) for w in want] and tokens.tolist() == sum(want, [])
    corpus = TokenCorpus.from_files(str(tmp_path / "c.bin"), str(tmp_path / "c.npy"))
    ds = GPTSampleDataset(corpus, seq_length=4, num_samples=3, seed=1)
    assert all(len(ds[i]) == 5 for i in range(len(ds)))
