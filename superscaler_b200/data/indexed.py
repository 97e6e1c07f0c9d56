"""Token datasets over a flat array of token ids with document boundaries (GPT-style language modelling).

Counterpart of the reference's GPT dataset machinery (runtime/megatron/data/gpt_dataset.py:_build_index_mappings,
runtime/megatron/data/blendable_dataset.py) reduced to what a training run needs:

  * `TokenCorpus`       : tokens (np.ndarray / np.memmap, any integer dtype) + document lengths;
  * `GPTSampleDataset`  : samples of seq_length + 1 consecutive tokens drawn from `num_epochs` shuffled passes over
                          the documents; three index arrays (document order, sample starts, sample order) built
                          once from a seed.  The sample-start index is built by the native helper
                          (`csrc_host/dataset_helpers.cpp`), with a pure-Python fallback of the same definition;
  * `BlendedDataset`    : weighted mixture of datasets with a deterministic interleaving;
  * `batches`           : pinned-memory global batches in the layout `Trainer.train_step` takes.
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Sequence

import numpy as np
import torch

try:  # built by `python -m superscaler_b200.build`
    from .. import _data_helpers as _native
except ImportError:  # pragma: no cover - the fallback below has the same semantics
    _native = None


class TokenCorpus:
    def __init__(self, tokens: np.ndarray, doc_lengths: Sequence[int]):
        self.tokens = tokens
        self.sizes = np.asarray(doc_lengths, dtype=np.int32)
        assert int(self.sizes.sum()) == len(tokens), "document lengths must cover the token array"
        self.doc_start = np.concatenate([[0], np.cumsum(self.sizes, dtype=np.int64)])

    @classmethod
    def from_files(cls, token_file: str, lengths_file: str, dtype=np.uint16) -> "TokenCorpus":
        return cls(np.memmap(token_file, dtype=dtype, mode="r"), np.load(lengths_file))

    def slice_docs(self, first: int, last: int) -> "TokenCorpus":
        """Documents [first, last) as a corpus of their own (a view of the same tokens)."""
        return TokenCorpus(self.tokens[self.doc_start[first]:self.doc_start[last]], self.sizes[first:last])


def split_bounds(spec: str, n: int) -> List[int]:
    """Document boundaries [0, a, b, n] of the train / validation / test parts for a weight string such as
    "949,50,1" (also "98/2", or one number = everything trains).  Each part gets round(weight share x n)
    documents and the rounding surplus is taken off all three upper boundaries, which is the reference's rule
    (get_train_valid_test_split_, runtime/megatron/data/dataset_utils.py:606-632)."""
    weights = [float(x) for x in spec.replace("/", ",").split(",") if x.strip()]
    weights = (weights + [0.0, 0.0])[:3]
    total = sum(weights)
    assert total > 0 and min(weights) >= 0, f"--split {spec!r}: weights must be non-negative, not all zero"
    bounds = [0]
    for w in weights:
        bounds.append(bounds[-1] + int(round(w / total * n)))
    surplus = bounds[-1] - n
    bounds = [0] + [b - surplus for b in bounds[1:]]
    assert bounds == sorted(bounds) and bounds[-1] == n and bounds[1] >= 0, f"--split {spec!r} leaves a part negative"
    return bounds


def build_sample_idx_py(sizes, doc_idx, seq_length: int, num_epochs: int, tokens_per_epoch: int) -> np.ndarray:
    """Reference definition of the sample-start index (see dataset_helpers.cpp)."""
    num_samples = (num_epochs * tokens_per_epoch - 1) // seq_length
    out = np.zeros((num_samples + 1, 2), dtype=np.int32)
    pos, offset = 0, 0
    for s in range(1, num_samples + 1):
        need = seq_length + 1
        while need > 0:
            left = int(sizes[doc_idx[pos]]) - offset
            if left >= need:
                offset += need - 1
                need = 0
            else:
                need -= left
                pos += 1
                offset = 0
        out[s] = (pos, offset)
    return out


def build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch) -> np.ndarray:
    if _native is not None:
        return _native.build_sample_idx(np.ascontiguousarray(sizes, dtype=np.int32),
                                        np.ascontiguousarray(doc_idx, dtype=np.int32), int(seq_length),
                                        int(num_epochs), int(tokens_per_epoch))
    return build_sample_idx_py(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch)


class GPTSampleDataset:
    def __init__(self, corpus: TokenCorpus, seq_length: int, num_samples: int, seed: int = 1234):
        self.corpus, self.seq_length = corpus, seq_length
        tokens_per_epoch = int(corpus.sizes.sum())
        num_epochs = 1
        while (num_epochs * tokens_per_epoch - 1) // seq_length < num_samples:
            num_epochs += 1
        rng = np.random.RandomState(seed)
        # every epoch is its own permutation of the documents
        self.doc_idx = np.concatenate([rng.permutation(len(corpus.sizes)) for _ in range(num_epochs)]).astype(np.int32)
        self.sample_idx = build_sample_idx(corpus.sizes, self.doc_idx, seq_length, num_epochs, tokens_per_epoch)
        self.shuffle_idx = rng.permutation(self.sample_idx.shape[0] - 1).astype(np.int64)
        self.num_samples = num_samples

    def __len__(self) -> int:
        return min(self.num_samples, len(self.shuffle_idx))

    def __getitem__(self, i: int) -> np.ndarray:
        """seq_length + 1 token ids (inputs = [:-1], labels = [1:])."""
        s = int(self.shuffle_idx[i])
        (p0, o0), (p1, o1) = self.sample_idx[s], self.sample_idx[s + 1]
        c = self.corpus
        if p0 == p1:
            a = c.doc_start[self.doc_idx[p0]]
            return np.asarray(c.tokens[a + o0: a + o1 + 1], dtype=np.int64)
        parts = [c.tokens[c.doc_start[self.doc_idx[p0]] + o0: c.doc_start[self.doc_idx[p0] + 1]]]
        for p in range(p0 + 1, p1):
            d = self.doc_idx[p]
            parts.append(c.tokens[c.doc_start[d]: c.doc_start[d + 1]])
        a = c.doc_start[self.doc_idx[p1]]
        parts.append(c.tokens[a: a + o1 + 1])
        return np.concatenate(parts).astype(np.int64)


class BlendedDataset:
    def __init__(self, datasets: List, weights: Sequence[float], size: int):
        w = np.asarray(weights, dtype=np.float64)
        w = w / w.sum()
        self.datasets = datasets
        self.dataset_index = np.zeros(size, dtype=np.uint8)
        self.sample_index = np.zeros(size, dtype=np.int64)
        if _native is not None:
            _native.build_blending_indices(self.dataset_index, self.sample_index, w, len(datasets), size)
        else:
            drawn = np.zeros(len(datasets), dtype=np.int64)
            for s in range(size):
                lag = w * max(s, 1) - drawn
                d = int(np.argmax(lag))
                self.dataset_index[s], self.sample_index[s] = d, drawn[d]
                drawn[d] += 1

    def __len__(self) -> int:
        return len(self.dataset_index)

    def __getitem__(self, i: int):
        d = self.datasets[int(self.dataset_index[i])]
        return d[int(self.sample_index[i]) % len(d)]


def batches(dataset, global_bs: int, steps: int, start: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """Global batches {ids, labels, loss_mask} in pinned memory, consecutive samples of `dataset`."""
    for it in range(steps):
        rows = np.stack([dataset[(start + it * global_bs + j) % len(dataset)] for j in range(global_bs)])
        t = torch.from_numpy(rows)
        out = {"ids": t[:, :-1].contiguous(), "labels": t[:, 1:].contiguous(),
               "loss_mask": torch.ones(rows.shape[0], rows.shape[1] - 1, dtype=torch.float32)}
        if torch.cuda.is_available():
            out = {k: v.pin_memory() for k, v in out.items()}
        yield out
