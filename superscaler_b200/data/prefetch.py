"""Batches prepared ahead of the training loop by worker threads.

A batch function here is a pure function of the iteration number (every dataset draws sample i from generators seeded
by (seed, epoch, i)), so batches can be built in any order and in parallel without changing what the run sees.  The
workers are threads: image decoding, numpy and the token gathers release the interpreter lock, and the training
thread spends its time waiting for the device.  Counterpart of the worker processes of the reference's data loader
(`--num-workers`, runtime/megatron/data/data_samplers.py:25-60).
"""
from __future__ import annotations

from concurrent.futures import Future, ThreadPoolExecutor
from typing import Callable, Dict, Optional


class Prefetcher:
    """`prefetcher(i)` returns `batch_fn(i)`; batches i + 1 ... i + depth are started in the background.  Attributes
    of the wrapped function (`valid`, `test`) stay reachable."""

    def __init__(self, batch_fn: Callable[[int], dict], workers: int = 2, depth: Optional[int] = None,
                 stop: Optional[int] = None):
        assert workers >= 1
        self.fn, self.stop = batch_fn, stop
        self.depth = workers if depth is None else depth
        self.pool = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="batch")
        self.pending: Dict[int, Future] = {}
        self.valid = getattr(batch_fn, "valid", None)
        self.test = getattr(batch_fn, "test", None)

    def _start(self, i: int) -> Future:
        if i not in self.pending:
            self.pending[i] = self.pool.submit(self.fn, i)
        return self.pending[i]

    def __call__(self, i: int) -> dict:
        fut = self._start(i)
        last = i + self.depth if self.stop is None else min(i + self.depth, self.stop - 1)
        for j in range(i + 1, last + 1):
            self._start(j)
        for j in [j for j in self.pending if j < i]:        # a caller that jumped ahead: drop what it skipped
            self.pending.pop(j).cancel()
        del self.pending[i]
        return fut.result()

    def close(self) -> None:
        for f in self.pending.values():
            f.cancel()
        self.pending.clear()
        self.pool.shutdown(wait=True)
