"""Sentence-level corpora and the datasets built on them: masked-LM samples (BERT style), span-corruption samples
(T5 style) and inverse-cloze blocks.

Counterpart of the reference's inherited Megatron data pipeline (runtime/megatron/data/dataset_utils.py,
bert_dataset.py, t5_dataset.py, ict_dataset.py and the index builders build_mapping / build_blocks_mapping of
data/helpers.cpp).  A sample is a run of whole consecutive sentences of one document chosen by the sentence map;
the maps are built by the native host helper (`csrc_host/dataset_helpers.cpp`), with Python definitions of the same
algorithm here (same splitmix64 stream, so both produce identical arrays).

  * `SentenceCorpus`                : flat token array + sentence lengths + first sentence of every document;
  * `build_mapping` / `build_blocks_mapping` : (first sentence, one past last, target length) rows / (first, one
                                      past last, document, block id) rows, shuffled;
  * `create_masked_lm_predictions`  : n-gram masking, BERT (80 / 10 / 10 replacement) or T5 (span) style;
  * `BertDataset`, `T5Dataset`, `InverseClozeDataset`;
  * `t5_batches`                    : global batches in the layout the T5 trainer takes (ids, dec_ids, labels,
                                      loss_mask, enc_lens).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

try:  # built by `python -m superscaler_b200.build`
    from .. import _data_helpers as _native
except ImportError:  # pragma: no cover - the definitions below have the same semantics
    _native = None

LONG_SENTENCE = 512
_M64 = (1 << 64) - 1


class SplitMix64:
    """The generator the native helper uses (so that Python and C++ draw the same stream)."""

    def __init__(self, seed: int):
        self.state = seed & _M64

    def next(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        return z ^ (z >> 31)


class SentenceCorpus:
    def __init__(self, tokens: np.ndarray, sentence_lengths: Sequence[int], doc_starts: Sequence[int],
                 title_lengths: Optional[Sequence[int]] = None):
        self.tokens = tokens
        self.sizes = np.asarray(sentence_lengths, dtype=np.int32)
        self.doc_starts = np.asarray(doc_starts, dtype=np.int64)   # D + 1 entries, last = number of sentences
        assert int(self.sizes.sum()) == len(tokens), "sentence lengths must cover the token array"
        assert self.doc_starts[0] == 0 and self.doc_starts[-1] == len(self.sizes)
        self.sent_start = np.concatenate([[0], np.cumsum(self.sizes, dtype=np.int64)])
        self.title_sizes = None if title_lengths is None else np.asarray(title_lengths, dtype=np.int32)

    def sentences(self, first: int, last: int) -> List[np.ndarray]:
        return [np.asarray(self.tokens[self.sent_start[i]:self.sent_start[i + 1]]) for i in range(first, last)]

    def slice_docs(self, first: int, last: int) -> "SentenceCorpus":
        """Documents [first, last) as a corpus of their own (a view of the same tokens)."""
        s0, s1 = int(self.doc_starts[first]), int(self.doc_starts[last])
        return SentenceCorpus(self.tokens[self.sent_start[s0]:self.sent_start[s1]], self.sizes[s0:s1],
                              self.doc_starts[first:last + 1] - s0,
                              None if self.title_sizes is None else self.title_sizes[first:last])


def _usable(sizes, first, last, min_sent) -> bool:
    return last - first >= min_sent and not (sizes[first:last] > LONG_SENTENCE).any()


def _shuffled(rows: List[Tuple[int, ...]], width: int, seed: int) -> np.ndarray:
    rng = SplitMix64(seed)
    for i in range(len(rows) - 1, 0, -1):
        j = rng.next() % (i + 1)
        rows[i], rows[j] = rows[j], rows[i]
    return np.asarray(rows, dtype=np.int64).reshape(len(rows), width)


def _draw_target(rng: SplitMix64, short_ratio: int, max_length: int) -> int:
    if short_ratio == 0:
        return max_length
    r = rng.next()
    if r % short_ratio == 0:
        return 2 + (r >> 20) % (max_length - 1)
    return max_length


def build_mapping_py(doc_starts, sizes, num_epochs, max_num_samples, max_seq_length, short_seq_prob, seed,
                     min_num_sent) -> np.ndarray:
    short_ratio = int(1.0 / short_seq_prob + 0.5) if short_seq_prob > 0 else 0
    rows: List[Tuple[int, ...]] = []
    rng = SplitMix64(seed)
    for _ in range(num_epochs):
        if len(rows) >= max_num_samples:
            break
        for d in range(len(doc_starts) - 1):
            first, last = int(doc_starts[d]), int(doc_starts[d + 1])
            if not _usable(sizes, first, last, min_num_sent):
                continue
            start, remain, length, count = first, last - first, 0, 0
            target = _draw_target(rng, short_ratio, max_seq_length)
            for i in range(first, last):
                length += int(sizes[i])
                count += 1
                remain -= 1
                if (length >= target and remain > 1 and count >= min_num_sent) or remain == 0:
                    rows.append((start, i + 1, target))
                    start, length, count = i + 1, 0, 0
                    target = _draw_target(rng, short_ratio, max_seq_length)
    return _shuffled(rows, 3, seed + 1)


def build_blocks_mapping_py(doc_starts, sizes, title_sizes, num_epochs, max_num_samples, max_seq_length, seed,
                            use_one_sent_blocks) -> np.ndarray:
    min_sent = 1 if use_one_sent_blocks else 2
    rows: List[Tuple[int, ...]] = []
    for _ in range(num_epochs):
        if len(rows) >= max_num_samples:
            break
        block_id = 0
        for d in range(len(doc_starts) - 1):
            first, last = int(doc_starts[d]), int(doc_starts[d + 1])
            if not _usable(sizes, first, last, min_sent):
                continue
            target = max_seq_length - int(title_sizes[d])
            start, remain, length, count = first, last - first, 0, 0
            for i in range(first, last):
                length += int(sizes[i])
                count += 1
                remain -= 1
                if (length >= target and remain >= min_sent and count >= min_sent) or remain == 0:
                    rows.append((start, i + 1, d, block_id))
                    block_id += 1
                    start, length, count = i + 1, 0, 0
    return _shuffled(rows, 4, seed + 1)


def build_mapping(corpus: SentenceCorpus, num_epochs: int, max_num_samples: int, max_seq_length: int,
                  short_seq_prob: float, seed: int, min_num_sent: int = 2) -> np.ndarray:
    args = (corpus.doc_starts, corpus.sizes, num_epochs, max_num_samples, max_seq_length, short_seq_prob, seed,
            min_num_sent)
    return _native.build_mapping(*args) if _native is not None else build_mapping_py(*args)


def build_blocks_mapping(corpus: SentenceCorpus, num_epochs: int, max_num_samples: int, max_seq_length: int,
                         seed: int, use_one_sent_blocks: bool = False) -> np.ndarray:
    assert corpus.title_sizes is not None, "block samples need the title length of every document"
    args = (corpus.doc_starts, corpus.sizes, corpus.title_sizes, num_epochs, max_num_samples, max_seq_length, seed,
            use_one_sent_blocks)
    return _native.build_blocks_mapping(*args) if _native is not None else build_blocks_mapping_py(*args)


# ---- masking -------------------------------------------------------------------------------------------

@dataclass
class MaskedSpan:
    positions: List[int]     # consecutive token positions
    labels: List[int]        # the original tokens there


def create_masked_lm_predictions(tokens: Sequence[int], vocab_size: int, mask_id: int, special_ids: Sequence[int],
                                 masked_lm_prob: float, max_predictions: int, rng: np.random.RandomState,
                                 style: str = "bert", max_ngrams: int = 3, geometric: bool = False):
    """Chooses n-gram spans covering about masked_lm_prob of the tokens (never a special token, never overlapping).

    style "bert": every chosen position becomes mask_id (80 %), stays (10 %) or becomes a random id (10 %);
    style "t5":   the tokens are left untouched and the spans are returned for sentinel replacement.
    Span lengths are drawn from a geometric distribution (p = 0.2, capped) when `geometric`, else with weight 1 / n.
    Returns (output tokens, masked positions, labels at those positions, spans sorted by position).
    (reference: create_masked_lm_predictions, runtime/megatron/data/dataset_utils.py:180-390)
    """
    out = list(tokens)
    special = set(special_ids)
    candidates = [i for i, t in enumerate(tokens) if t not in special]
    want = min(int(max_predictions), max(1, int(round(len(tokens) * masked_lm_prob))))
    if not candidates or want <= 0:
        return out, [], [], []
    lengths = np.arange(1, max_ngrams + 1)
    weights = 1.0 / lengths
    weights /= weights.sum()
    order = list(candidates)
    rng.shuffle(order)
    cand_set = set(candidates)
    taken: set = set()
    spans: List[MaskedSpan] = []
    covered = 0
    for start in order:
        if covered >= want:
            break
        n = min(int(rng.geometric(0.2)), max_ngrams) if geometric else int(rng.choice(lengths, p=weights))
        n = min(n, want - covered)
        pos = []
        for i in range(start, start + n):
            if i not in cand_set or i in taken:
                break
            pos.append(i)
        if not pos:
            continue
        # keep one untouched token between neighbouring spans so that sentinels never touch
        if (pos[0] - 1) in taken or (pos[-1] + 1) in taken:
            continue
        taken.update(pos)
        covered += len(pos)
        spans.append(MaskedSpan(pos, [int(tokens[i]) for i in pos]))
    spans.sort(key=lambda s: s.positions[0])
    positions = [i for s in spans for i in s.positions]
    labels = [l for s in spans for l in s.labels]
    if style == "bert":
        for i in positions:
            r = rng.random_sample()
            if r < 0.8:
                out[i] = mask_id
            elif r < 0.9:
                out[i] = int(rng.randint(0, vocab_size))
    elif style != "t5":
        raise ValueError(style)
    return out, positions, labels, spans


@dataclass
class SpecialTokens:
    cls: int
    sep: int
    mask: int
    pad: int
    bos: Optional[int] = None
    eos: Optional[int] = None
    sentinels: Tuple[int, ...] = ()


class _MappedDataset:
    def __init__(self, corpus: SentenceCorpus, num_samples: int, max_seq_length: int, short_seq_prob: float,
                 seed: int, min_num_sent: int, reserve: int):
        self.corpus, self.seed, self.max_seq_length = corpus, seed, max_seq_length
        per_epoch = max(1, len(build_mapping(corpus, 1, 1 << 62, max_seq_length - reserve, short_seq_prob, seed,
                                             min_num_sent)))
        epochs = (num_samples + per_epoch - 1) // per_epoch
        self.mapping = build_mapping(corpus, epochs, num_samples, max_seq_length - reserve, short_seq_prob, seed,
                                     min_num_sent)

    def __len__(self) -> int:
        return len(self.mapping)

    def _rng(self, i: int) -> np.random.RandomState:
        return np.random.RandomState((self.seed + i) % (1 << 32))


class BertDataset(_MappedDataset):
    """[CLS] A [SEP] B [SEP] samples with masked-LM labels and the sentence-order flag
    (reference: runtime/megatron/data/bert_dataset.py:build_training_sample)."""

    def __init__(self, corpus: SentenceCorpus, tokens: SpecialTokens, vocab_size: int, num_samples: int,
                 max_seq_length: int, masked_lm_prob: float = 0.15, short_seq_prob: float = 0.1, seed: int = 1234,
                 binary_head: bool = True):
        super().__init__(corpus, num_samples, max_seq_length, short_seq_prob, seed, 2 if binary_head else 1, 3)
        self.tok, self.vocab_size, self.masked_lm_prob, self.binary_head = tokens, vocab_size, masked_lm_prob, binary_head

    def __getitem__(self, i: int) -> Dict[str, np.ndarray]:
        first, last, target = (int(x) for x in self.mapping[i])
        rng = self._rng(i)
        sents = self.corpus.sentences(first, last)
        if self.binary_head and len(sents) > 1:
            cut = int(rng.randint(1, len(sents)))
            a = [t for s in sents[:cut] for t in s]
            b = [t for s in sents[cut:] for t in s]
            is_random = bool(rng.random_sample() < 0.5)
            if is_random:
                a, b = b, a
        else:
            a, b, is_random = [t for s in sents for t in s], [], False
        truncated = len(a) + len(b) > target
        while len(a) + len(b) > target:     # trim the longer segment from a random end
            side = a if len(a) > len(b) else b
            if rng.random_sample() < 0.5:
                del side[0]
            else:
                side.pop()
        t = self.tok
        text = [t.cls] + [int(x) for x in a] + [t.sep]
        types = [0] * len(text)
        if b:
            text += [int(x) for x in b] + [t.sep]
            types += [1] * (len(b) + 1)
        text, positions, labels, _ = create_masked_lm_predictions(
            text, self.vocab_size, t.mask, (t.cls, t.sep), self.masked_lm_prob,
            self.masked_lm_prob * self.max_seq_length, rng, style="bert", max_ngrams=3)
        n, L = len(text), self.max_seq_length
        out_labels = np.full(L, -1, dtype=np.int64)
        loss_mask = np.zeros(L, dtype=np.int64)
        out_labels[positions] = labels
        loss_mask[positions] = 1
        pad = [t.pad] * (L - n)
        return {"text": np.asarray(text + pad, dtype=np.int64), "types": np.asarray(types + pad, dtype=np.int64),
                "labels": out_labels, "is_random": int(is_random), "loss_mask": loss_mask,
                "padding_mask": np.asarray([1] * n + [0] * (L - n), dtype=np.int64), "truncated": int(truncated)}


class T5Dataset(_MappedDataset):
    """Span corruption: every masked span becomes one sentinel in the encoder input; the decoder sees
    [bos] sentinel span sentinel span ... and predicts the same sequence shifted, closed by [eos]
    (reference: runtime/megatron/data/t5_dataset.py:build_training_sample, pad_and_convert_to_numpy)."""

    def __init__(self, corpus: SentenceCorpus, tokens: SpecialTokens, vocab_size: int, num_samples: int,
                 max_seq_length: int, max_seq_length_dec: int, masked_lm_prob: float = 0.15,
                 short_seq_prob: float = 0.0, seed: int = 1234):
        super().__init__(corpus, num_samples, max_seq_length, short_seq_prob, seed, 1, 2)
        assert tokens.bos is not None and tokens.eos is not None and tokens.sentinels
        self.tok, self.vocab_size, self.masked_lm_prob = tokens, vocab_size, masked_lm_prob
        self.max_seq_length_dec = max_seq_length_dec

    def __getitem__(self, i: int) -> Dict[str, np.ndarray]:
        first, last, target = (int(x) for x in self.mapping[i])
        rng = self._rng(i)
        flat = [int(t) for s in self.corpus.sentences(first, last) for t in s]
        truncated = len(flat) > target
        flat = flat[:target]
        t = self.tok
        # the decoder sequence holds one sentinel per span plus the span tokens plus [bos]
        budget = min(self.masked_lm_prob * target, (self.max_seq_length_dec - 2) // 2, len(t.sentinels))
        _, _, _, spans = create_masked_lm_predictions(flat, self.vocab_size, t.mask, (t.cls, t.sep),
                                                      self.masked_lm_prob, max(1, budget), rng, style="t5",
                                                      max_ngrams=10, geometric=True)
        spans = spans[:len(t.sentinels)]
        enc: List[int] = []
        dec_in, dec_out = [t.bos], []
        at = 0
        for sentinel, span in zip(t.sentinels, spans):
            enc += flat[at:span.positions[0]] + [sentinel]
            dec_in += [sentinel] + span.labels
            dec_out += [sentinel] + span.labels
            at = span.positions[-1] + 1
        enc += flat[at:]
        dec_out.append(t.eos)
        L, Ld = self.max_seq_length, self.max_seq_length_dec
        assert len(enc) <= L and len(dec_in) <= Ld, "span budget exceeded the decoder length"
        n, nd = len(enc), len(dec_in)
        return {"text_enc": np.asarray(enc + [t.pad] * (L - n), dtype=np.int64),
                "text_dec": np.asarray(dec_in + [t.pad] * (Ld - nd), dtype=np.int64),
                "labels": np.asarray(dec_out + [-1] * (Ld - nd), dtype=np.int64),
                "loss_mask": np.asarray([1] * nd + [0] * (Ld - nd), dtype=np.int64),
                "enc_len": n, "dec_len": nd, "truncated": int(truncated)}


class InverseClozeDataset:
    """(query sentence, remaining block) pairs for retrieval pre-training; the query stays inside its block with
    probability `query_in_block_prob` (reference: runtime/megatron/data/ict_dataset.py)."""

    def __init__(self, corpus: SentenceCorpus, titles: Sequence[np.ndarray], tokens: SpecialTokens, num_samples: int,
                 max_seq_length: int, query_in_block_prob: float = 0.1, seed: int = 1234,
                 use_one_sent_blocks: bool = False):
        self.corpus, self.titles, self.tok, self.seed = corpus, titles, tokens, seed
        self.max_seq_length, self.query_in_block_prob = max_seq_length, query_in_block_prob
        one = build_blocks_mapping(corpus, 1, 1 << 62, max_seq_length, seed, use_one_sent_blocks)
        epochs = (num_samples + max(1, len(one)) - 1) // max(1, len(one))
        self.mapping = build_blocks_mapping(corpus, epochs, num_samples, max_seq_length, seed, use_one_sent_blocks)

    def __len__(self) -> int:
        return len(self.mapping)

    def _pad(self, ids: List[int]) -> Tuple[np.ndarray, np.ndarray]:
        L = self.max_seq_length
        ids = ids[:L]
        return (np.asarray(ids + [self.tok.pad] * (L - len(ids)), dtype=np.int64),
                np.asarray([1] * len(ids) + [0] * (L - len(ids)), dtype=np.int64))

    def __getitem__(self, i: int) -> Dict[str, np.ndarray]:
        first, last, doc, block = (int(x) for x in self.mapping[i])
        rng = np.random.RandomState((self.seed + i) % (1 << 32))
        sents = [list(map(int, s)) for s in self.corpus.sentences(first, last)]
        q = int(rng.randint(0, len(sents)))
        query = sents[q]
        if len(sents) > 1 and rng.random_sample() >= self.query_in_block_prob:
            sents = sents[:q] + sents[q + 1:]
        t = self.tok
        title = list(map(int, self.titles[doc]))
        body = [x for s in sents for x in s][: self.max_seq_length - 3 - len(title)]
        q_ids, q_mask = self._pad([t.cls] + query[: self.max_seq_length - 2] + [t.sep])
        b_ids, b_mask = self._pad([t.cls] + title + [t.sep] + body + [t.sep])
        return {"query_tokens": q_ids, "query_pad_mask": q_mask, "block_tokens": b_ids, "block_pad_mask": b_mask,
                "block_data": np.asarray([first, last, doc, block], dtype=np.int64)}


def bert_batch_of(dataset: BertDataset, indices: Sequence[int]) -> Dict[str, torch.Tensor]:
    """One global batch for the BERT trainer: ids, token types, the number of real tokens per sample, masked-LM
    labels (-1 where nothing is predicted) with their loss mask, and the sentence-order flag."""
    rows = [dataset[int(i) % len(dataset)] for i in indices]
    out = {"ids": torch.from_numpy(np.stack([r["text"] for r in rows])),
           "types": torch.from_numpy(np.stack([r["types"] for r in rows])),
           "enc_lens": torch.tensor([int(r["padding_mask"].sum()) for r in rows], dtype=torch.int32),
           "labels": torch.from_numpy(np.stack([r["labels"] for r in rows])),
           "loss_mask": torch.from_numpy(np.stack([r["loss_mask"] for r in rows]).astype(np.float32)),
           "nsp": torch.tensor([r["is_random"] for r in rows], dtype=torch.int64)}
    if torch.cuda.is_available():
        out = {k: v.pin_memory() for k, v in out.items()}
    return out


def t5_batches(dataset: T5Dataset, global_bs: int, steps: int, start: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """Global batches for the T5 trainer: encoder ids, decoder ids, labels (padding positions 0 with loss_mask 0)
    and the number of real encoder tokens per sample, in pinned memory."""
    for it in range(steps):
        rows = [dataset[(start + it * global_bs + j) % len(dataset)] for j in range(global_bs)]
        labels = np.stack([r["labels"] for r in rows])
        out = {"ids": torch.from_numpy(np.stack([r["text_enc"] for r in rows])),
               "dec_ids": torch.from_numpy(np.stack([r["text_dec"] for r in rows])),
               "labels": torch.from_numpy(np.where(labels < 0, 0, labels)),
               "loss_mask": torch.from_numpy(np.stack([r["loss_mask"] for r in rows]).astype(np.float32)),
               "enc_lens": torch.tensor([r["enc_len"] for r in rows], dtype=torch.int32)}
        if torch.cuda.is_available():
            out = {k: v.pin_memory() for k, v in out.items()}
        yield out
