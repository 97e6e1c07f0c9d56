"""Dataset index builders: the native helper against the Python definition, and end-to-end sample extraction."""
import numpy as np
import pytest

from superscaler_b200.data import indexed


def _corpus(n_docs=50, seed=0):
    rng = np.random.RandomState(seed)
    sizes = rng.randint(1, 40, size=n_docs)
    tokens = np.arange(int(sizes.sum()), dtype=np.int32)     # token value = position in the corpus
    return indexed.TokenCorpus(tokens, sizes)


@pytest.mark.parametrize("seq", [1, 7, 32, 100])
def test_native_sample_idx_matches_python_definition(seq):
    if indexed._native is None:
        pytest.skip("host helpers not built")
    c = _corpus()
    rng = np.random.RandomState(1)
    epochs = 3
    doc_idx = np.concatenate([rng.permutation(len(c.sizes)) for _ in range(epochs)]).astype(np.int32)
    tpe = int(c.sizes.sum())
    a = indexed._native.build_sample_idx(c.sizes, doc_idx, seq, epochs, tpe)
    b = indexed.build_sample_idx_py(c.sizes, doc_idx, seq, epochs, tpe)
    assert a.shape == b.shape and np.array_equal(a, b)


def test_samples_are_contiguous_stream_windows():
    c = _corpus()
    ds = indexed.GPTSampleDataset(c, seq_length=16, num_samples=200, seed=3)
    # the token stream in document order doc_idx
    stream = np.concatenate([c.tokens[c.doc_start[d]: c.doc_start[d + 1]] for d in ds.doc_idx])
    assert len(ds) == 200
    for i in range(0, 200, 7):
        s = int(ds.shuffle_idx[i])
        want = stream[s * 16: s * 16 + 17]
        got = ds[i]
        assert got.shape == (17,) and np.array_equal(got, want)


def test_blended_dataset_follows_weights():
    a, b = list(range(1000)), list(range(1000, 2000))
    bl = indexed.BlendedDataset([a, b], [0.75, 0.25], 400)
    counts = np.bincount(bl.dataset_index, minlength=2)
    assert abs(counts[0] - 300) <= 1 and abs(counts[1] - 100) <= 1
    assert bl[0] in a + b
    # running sample numbers inside each dataset are consecutive
    for d in (0, 1):
        idx = bl.sample_index[bl.dataset_index == d]
        assert np.array_equal(idx, np.arange(len(idx)))


def test_batches_layout():
    c = _corpus()
    ds = indexed.GPTSampleDataset(c, seq_length=8, num_samples=64, seed=0)
    batch = next(indexed.batches(ds, global_bs=4, steps=1))
    assert batch["ids"].shape == (4, 8) and batch["labels"].shape == (4, 8)
    assert (batch["ids"][:, 1:] == batch["labels"][:, :-1]).all()


def test_samplers_resume_and_shard():
    from superscaler_b200.data.samplers import (SequentialBatchSampler, ShuffledBatchSampler, build_data_loader,
                                                stack_samples)
    s = SequentialBatchSampler(22, 4)
    all_b = list(s)
    assert len(all_b) == 5 and all_b[0] == [0, 1, 2, 3] and all_b[-1] == [16, 17, 18, 19] and s.consumed == 20
    assert list(SequentialBatchSampler(22, 4, consumed_samples=8))[0] == [8, 9, 10, 11]
    assert list(SequentialBatchSampler(22, 4, drop_last=False))[-1] == [20, 21]
    assert list(SequentialBatchSampler(22, 4, rows=slice(2, 4)))[1] == [6, 7]
    a = ShuffledBatchSampler(22, 4, seed=3, epochs=2)
    seq = list(a)
    assert len(seq) == 10
    assert len(set(sum(seq[:5], []))) == 20 and len(set(sum(seq[5:], []))) == 20 and seq[:5] != seq[5:]
    b = ShuffledBatchSampler(22, 4, seed=3, consumed_samples=12, epochs=2)
    assert list(b) == seq[3:]
    import numpy as np
    data = [np.arange(i, i + 9) for i in range(22)]
    loader = build_data_loader(data, SequentialBatchSampler(22, 4), stack_samples)
    first = next(iter(loader))
    assert first["ids"].shape == (4, 8) and (first["labels"][:, :-1] == first["ids"][:, 1:]).all()
