"""Region timers on CUDA events: start / stop only record events on the current stream; elapsed times are read
when a log line is produced, so the measured path contains no host synchronisation (the reference's _Timer
calls torch.cuda.synchronize() on every start and stop when PROFILING=1, runtime/megatron/global_vars.py:208-224).
On CPU tensors the timers fall back to the wall clock."""
from __future__ import annotations

import time
from typing import Dict, List

import torch


class _EventTimer:
    def __init__(self, name: str, cuda: bool):
        self.name, self.cuda = name, cuda
        self.pairs: List[tuple] = []
        self._open = None
        self.wall = 0.0

    def start(self):
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._open = e
        else:
            self._open = time.perf_counter()

    def stop(self):
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.pairs.append((self._open, e))
        else:
            self.wall += (time.perf_counter() - self._open) * 1000.0
        self._open = None

    def elapsed_ms(self, reset: bool = True) -> float:
        if self.cuda:
            if self.pairs:
                self.pairs[-1][1].synchronize()
            t = sum(a.elapsed_time(b) for a, b in self.pairs)
            if reset:
                self.pairs = []
            return t
        t = self.wall
        if reset:
            self.wall = 0.0
        return t


class Timers:
    def __init__(self, cuda: bool):
        self.cuda = cuda
        self.timers: Dict[str, _EventTimer] = {}

    def __call__(self, name: str) -> _EventTimer:
        if name not in self.timers:
            self.timers[name] = _EventTimer(name, self.cuda)
        return self.timers[name]

    def row(self, names, normalizer: float = 1.0, reset: bool = True) -> Dict[str, float]:
        return {n: self.timers[n].elapsed_ms(reset) / normalizer for n in names if n in self.timers}
