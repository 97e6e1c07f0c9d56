"""Guard words around device buffers that other GPUs (or asynchronous copy engines) write into.

A kernel that pushes one tile too many into a peer's buffer, or a flag table indexed with the wrong stride, corrupts
whatever the allocator placed next to it, and the damage shows up steps later somewhere else.  With guards, the
payload is carved out of a slightly larger allocation whose first and last `guard_bytes` hold a fixed bit pattern;
`check()` compares them on the host side (one small device-to-host copy: call it where the host synchronises anyway:
when the loss is read, before a checkpoint is written) and names the first overwritten word.

`parallel/symm.py` places guards around its symmetric buffers when SSB_CANARIES=1 (off by default: the pattern check
costs a synchronisation, and the payload then starts 256 bytes into the allocation).  Together with the bitwise replay
of a run under `--deterministic` and the host model of the epoch-flag protocol (`parallel/flag_protocol.py`) this is
the race / overrun detection of the framework; the reference has none (it relies on NCCL's own checks).
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

PATTERN = 0x5AFEC0DE                                                          # fits a signed 32-bit word
GUARD_BYTES = 256                                                             # keeps the payload 256-byte aligned


class GuardedBuffer:
    """`raw` = [guard | payload | guard] in one allocation of `dtype`; `body` is the payload view."""

    def __init__(self, numel: int, dtype: torch.dtype, device, alloc: Optional[Callable[..., torch.Tensor]] = None,
                 guard_bytes: int = GUARD_BYTES, name: str = "buffer"):
        esize = torch.empty((), dtype=dtype).element_size()
        assert guard_bytes % 4 == 0 and guard_bytes % esize == 0
        self.name, self.numel, self.guard_elems = name, numel, guard_bytes // esize
        pad = (-numel * esize) % 4                      # the trailing guard is read as 32-bit words
        self.tail_pad_elems = pad // esize if pad % esize == 0 else 0
        total = numel + 2 * self.guard_elems + self.tail_pad_elems
        self.raw = (alloc or torch.empty)(total, dtype=dtype, device=device)
        self.body = self.raw[self.guard_elems:self.guard_elems + numel]
        self.arm()

    def _guards(self):
        lead = self.raw[:self.guard_elems].view(torch.int32)
        start = self.guard_elems + self.numel + self.tail_pad_elems
        trail = self.raw[start:start + self.guard_elems].view(torch.int32)
        return lead, trail

    def arm(self) -> None:
        for g in self._guards():
            g.fill_(PATTERN)

    @property
    def body_offset_bytes(self) -> int:
        return self.guard_elems * self.raw.element_size()

    def check(self) -> List[str]:
        """Empty when both guards are intact; otherwise one line per damaged guard naming the first bad word."""
        out = []
        for where, g in zip(("in front of", "behind"), self._guards()):
            bad = (g != PATTERN).nonzero()
            if bad.numel():
                k = int(bad[0])
                out.append(f"{self.name}: guard word {k} {where} the payload holds {int(g[k]) & 0xffffffff:#010x} "
                           f"({int(bad.numel())} of {g.numel()} words overwritten)")
        return out


class GuardRegistry:
    """All guarded buffers of a process; `check()` gathers their reports."""

    def __init__(self):
        self.buffers: List[GuardedBuffer] = []

    def add(self, buf: GuardedBuffer) -> GuardedBuffer:
        self.buffers.append(buf)
        return buf

    def check(self) -> List[str]:
        return [line for b in self.buffers for line in b.check()]


REGISTRY = GuardRegistry()
