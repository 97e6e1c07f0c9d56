"""Sentence maps (native helper against the Python definition), masking and the BERT / T5 / inverse-cloze samples
(reference: runtime/megatron/data/helpers.cpp build_mapping / build_blocks_mapping, dataset_utils.py,
bert_dataset.py, t5_dataset.py, ict_dataset.py)."""
import numpy as np
import pytest

from superscaler_b200.data import sentences as S


def _corpus(seed=0, docs=40, title=False):
    rng = np.random.RandomState(seed)
    sizes, starts, titles = [], [0], []
    for d in range(docs):
        n = int(rng.randint(0, 9))            # empty and one-sentence documents occur
        lens = rng.randint(3, 40, size=n).tolist()
        if d == 7 and n:
            lens[0] = 600                     # a document with an over-long sentence is skipped
        sizes += lens
        starts.append(len(sizes))
        titles.append(int(rng.randint(2, 6)))
    tokens = rng.randint(10, 800, size=int(np.sum(sizes))).astype(np.int32)
    return S.SentenceCorpus(tokens, sizes, starts, titles if title else None)


@pytest.mark.skipif(S._native is None, reason="host helper not built")
@pytest.mark.parametrize("short_prob,min_sent", [(0.0, 2), (0.1, 2), (0.5, 1)])
def test_native_sentence_map_equals_python_definition(short_prob, min_sent):
    c = _corpus()
    args = (c.doc_starts, c.sizes, 3, 10 ** 9, 64, short_prob, 1234, min_sent)
    a, b = S._native.build_mapping(*args), S.build_mapping_py(*args)
    assert a.shape == b.shape and a.shape[1] == 3 and len(a) > 20 and (a == b).all()


@pytest.mark.skipif(S._native is None, reason="host helper not built")
def test_native_block_map_equals_python_definition():
    c = _corpus(title=True)
    for one in (False, True):
        args = (c.doc_starts, c.sizes, c.title_sizes, 2, 10 ** 9, 48, 77, one)
        a, b = S._native.build_blocks_mapping(*args), S.build_blocks_mapping_py(*args)
        assert a.shape == b.shape and a.shape[1] == 4 and (a == b).all()


def test_sentence_map_covers_each_usable_document_once_per_epoch():
    c = _corpus()
    m = S.build_mapping_py(c.doc_starts, c.sizes, 1, 10 ** 9, 64, 0.0, 5, 2)
    covered = np.zeros(len(c.sizes), dtype=np.int64)
    for first, last, target in m:
        assert last > first and target == 64
        covered[first:last] += 1
    for d in range(len(c.doc_starts) - 1):
        f, l = c.doc_starts[d], c.doc_starts[d + 1]
        usable = l - f >= 2 and not (c.sizes[f:l] > 512).any()
        assert (covered[f:l] == (1 if usable else 0)).all()
    # a stop at max_num_samples happens at an epoch boundary
    few = S.build_mapping_py(c.doc_starts, c.sizes, 5, len(m) + 1, 64, 0.0, 5, 2)
    assert len(few) == 2 * len(m)


def test_masking_styles():
    rng = np.random.RandomState(3)
    toks = [1] + list(range(100, 180)) + [2]
    out, pos, labels, spans = S.create_masked_lm_predictions(toks, 1000, 3, (1, 2), 0.15, 20, rng, style="bert")
    assert 1 <= len(pos) <= 12 and all(toks[p] == l for p, l in zip(pos, labels))
    assert out[0] == 1 and out[-1] == 2 and all(out[i] == toks[i] for i in range(len(toks)) if i not in pos)
    assert sum(out[p] == 3 for p in pos) >= len(pos) // 2
    out, pos, labels, spans = S.create_masked_lm_predictions(toks, 1000, 3, (1, 2), 0.15, 20, rng, style="t5",
                                                             max_ngrams=10, geometric=True)
    assert out == toks and spans == sorted(spans, key=lambda s: s.positions[0])
    flat = [p for s in spans for p in s.positions]
    assert flat == pos and len(set(flat)) == len(flat)
    for a, b in zip(spans, spans[1:]):
        assert b.positions[0] - a.positions[-1] >= 2     # sentinels never touch


def test_bert_samples():
    c = _corpus(1)
    tok = S.SpecialTokens(cls=1, sep=2, mask=3, pad=0)
    ds = S.BertDataset(c, tok, 1000, num_samples=50, max_seq_length=64, seed=11)
    assert len(ds) >= 50
    seen_random = set()
    for i in range(50):
        s = ds[i]
        n = int(s["padding_mask"].sum())
        assert s["text"].shape == (64,) and s["text"][0] == 1 and s["text"][n - 1] == 2 and (s["text"][n:] == 0).all()
        assert (s["labels"][s["loss_mask"] == 0] == -1).all() and (s["labels"][s["loss_mask"] == 1] >= 10).all()
        assert s["loss_mask"].sum() >= 1 and set(np.unique(s["types"][:n])) <= {0, 1}
        seen_random.add(s["is_random"])
        again = ds[i]
        assert all((again[k] == s[k]).all() if isinstance(s[k], np.ndarray) else again[k] == s[k] for k in s)
    assert seen_random == {0, 1}


def test_t5_samples_reconstruct_the_text():
    c = _corpus(2)
    sentinels = tuple(range(900, 880, -1))
    tok = S.SpecialTokens(cls=1, sep=2, mask=3, pad=0, bos=4, eos=5, sentinels=sentinels)
    ds = S.T5Dataset(c, tok, 1000, num_samples=30, max_seq_length=64, max_seq_length_dec=32, seed=5)
    for i in range(30):
        s = ds[i]
        enc = s["text_enc"][: s["enc_len"]].tolist()
        dec_in = s["text_dec"][: s["dec_len"]].tolist()
        labels = s["labels"][: s["dec_len"]].tolist()
        assert dec_in[0] == 4 and labels[-1] == 5 and dec_in[1:] == labels[:-1]
        assert (s["labels"][s["dec_len"]:] == -1).all() and s["loss_mask"].sum() == s["dec_len"]
        # splice the spans back into the encoder text
        spans, cur = {}, None
        for t in labels[:-1]:
            if t in sentinels:
                cur = t
                spans[cur] = []
            else:
                spans[cur].append(t)
        rebuilt = []
        for t in enc:
            rebuilt += spans[t] if t in sentinels else [t]
        first, last, target = (int(x) for x in ds.mapping[i])
        original = [int(x) for sent in c.sentences(first, last) for x in sent][:target]
        assert rebuilt == original
    b = next(S.t5_batches(ds, 4, 1))
    assert b["ids"].shape == (4, 64) and b["dec_ids"].shape == (4, 32) and b["enc_lens"].dtype.is_floating_point is False
    assert (b["labels"] >= 0).all() and b["loss_mask"].sum() > 0


def test_inverse_cloze_blocks():
    c = _corpus(3, title=True)
    titles = [np.arange(10, 10 + n) for n in c.title_sizes]
    tok = S.SpecialTokens(cls=1, sep=2, mask=3, pad=0)
    ds = S.InverseClozeDataset(c, titles, tok, num_samples=20, max_seq_length=64, seed=9)
    ids = set()
    for i in range(len(ds)):
        s = ds[i]
        first, last, doc, block = s["block_data"]
        assert c.doc_starts[doc] <= first < last <= c.doc_starts[doc + 1]
        assert s["query_tokens"][0] == 1 and s["block_tokens"][0] == 1 and s["block_pad_mask"].sum() <= 64
        ids.add(int(block))
    assert len(ids) > 5


def test_t5_trains_on_span_corruption_batches():
    from superscaler_b200.runtime.trainer import Trainer
    from helpers import tiny_t5_plan
    c = _corpus(4, docs=60)
    sentinels = tuple(range(250, 230, -1))
    tok = S.SpecialTokens(cls=1, sep=2, mask=3, pad=0, bos=4, eos=5, sentinels=sentinels)
    c.tokens = (c.tokens % 200 + 10).astype(np.int32)      # vocabulary of the tiny model
    ds = S.T5Dataset(c, tok, 256, num_samples=16, max_seq_length=64, max_seq_length_dec=32, seed=5)
    t = Trainer(tiny_t5_plan(), model_overrides=dict(hidden_dropout=0.0, attention_dropout=0.0), lr_warmup_steps=0,
                device="cpu", lr=2e-3)
    losses = [t.loss_value(t.train_step(b)) for b in S.t5_batches(ds, 4, 6)]
    assert all(np.isfinite(losses)) and min(losses[3:]) < losses[0]
