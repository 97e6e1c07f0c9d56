"""Batch samplers that can resume from a number of consumed samples, and the loader around them.

Counterpart of the reference's MegatronPretrainingSampler ("single") and MegatronPretrainingRandomSampler
("cyclic") with build_pretraining_data_loader (runtime/megatron/data/data_samplers.py:25-157).  The trainer takes
one GLOBAL batch per step and every rank slices the rows its first / last op needs, so a sampler yields the indices
of a whole global batch; `rows` narrows them to a slice for callers that load only their own shard.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterator, List, Optional

import numpy as np
import torch


class SequentialBatchSampler:
    """Indices consumed, consumed + 1, ... in global batches; the last partial batch is dropped unless asked for."""

    def __init__(self, total_samples: int, global_batch_size: int, consumed_samples: int = 0,
                 drop_last: bool = True, rows: Optional[slice] = None):
        assert total_samples > 0 and global_batch_size > 0 and 0 <= consumed_samples < total_samples
        self.total, self.bs, self.consumed, self.drop_last, self.rows = \
            total_samples, global_batch_size, consumed_samples, drop_last, rows

    def __len__(self) -> int:
        left = self.total - self.consumed
        return left // self.bs if self.drop_last else -(-left // self.bs)

    def __iter__(self) -> Iterator[List[int]]:
        at = self.consumed
        while at + self.bs <= self.total or (not self.drop_last and at < self.total):
            batch = list(range(at, min(at + self.bs, self.total)))
            at += self.bs
            self.consumed = min(at, self.total)
            yield batch[self.rows] if self.rows is not None else batch


class ShuffledBatchSampler:
    """Endless passes over a fresh permutation per epoch (seed + epoch); the tail of an epoch that does not fill a
    global batch is dropped.  Resuming with `consumed_samples` continues inside the same epoch's permutation."""

    def __init__(self, total_samples: int, global_batch_size: int, consumed_samples: int = 0, seed: int = 0,
                 rows: Optional[slice] = None, epochs: Optional[int] = None):
        assert total_samples >= global_batch_size > 0
        self.total, self.bs, self.consumed, self.seed, self.rows, self.epochs = \
            total_samples, global_batch_size, consumed_samples, seed, rows, epochs
        self.per_epoch = total_samples // global_batch_size * global_batch_size

    def __iter__(self) -> Iterator[List[int]]:
        while self.epochs is None or self.consumed < self.epochs * self.per_epoch:
            epoch, at = divmod(self.consumed, self.per_epoch)
            assert at % self.bs == 0, "consumed samples must be a multiple of the global batch size"
            perm = np.random.RandomState((self.seed + epoch) % (1 << 32)).permutation(self.total)[: self.per_epoch]
            batch = perm[at:at + self.bs].tolist()
            self.consumed += self.bs
            yield batch[self.rows] if self.rows is not None else batch


def stack_samples(samples: List) -> Dict[str, torch.Tensor]:
    """Collates dict samples (numpy arrays / ints per key) or raw token rows of seq_length + 1 into a batch."""
    if isinstance(samples[0], dict):
        return {k: torch.from_numpy(np.stack([np.asarray(s[k]) for s in samples])) for k in samples[0]}
    t = torch.from_numpy(np.stack(samples).astype(np.int64))
    return {"ids": t[:, :-1].contiguous(), "labels": t[:, 1:].contiguous(),
            "loss_mask": torch.ones(t.shape[0], t.shape[1] - 1, dtype=torch.float32)}


def build_data_loader(dataset, sampler, collate: Callable = stack_samples, num_workers: int = 0):
    """torch DataLoader over a batch sampler; batches land in pinned memory when a GPU is present."""
    return torch.utils.data.DataLoader(dataset, batch_sampler=sampler, num_workers=num_workers, collate_fn=collate,
                                       pin_memory=torch.cuda.is_available())
