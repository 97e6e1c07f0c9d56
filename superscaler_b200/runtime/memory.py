"""Pre-allocated scratch buffers and memory reports.

`MemoryBuffer` hands out views of one flat allocation (bump allocation, reset per step); `RingMemBuffer` cycles
through several of them (reference: runtime/megatron/memory.py:26-145, used there for distributed checkpointed
activations; here `runtime/stage.py` keeps those shares as plain allocations and these classes serve user code).  `report_memory` / `debug_mem_report` are the reference's utils.report_memory and debug_mem_report
(runtime/megatron/utils.py): allocator statistics in MB, and a walk over the live tensors grouped by shape."""
from __future__ import annotations

import gc
from typing import Dict, List, Tuple

import torch

_BUFFERS: Dict[str, "MemoryBuffer"] = {}


def allocate_mem_buff(name: str, numel: int, dtype: torch.dtype, track_usage: bool = False, device=None):
    assert name not in _BUFFERS, f"memory buffer {name} already allocated"
    _BUFFERS[name] = MemoryBuffer(name, numel, dtype, track_usage, device)
    return _BUFFERS[name]


def get_mem_buff(name: str) -> "MemoryBuffer":
    return _BUFFERS[name]


class MemoryBuffer:
    def __init__(self, name: str, numel: int, dtype: torch.dtype, track_usage: bool = False, device=None):
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        self.name, self.numel, self.dtype, self.track_usage = name, numel, dtype, track_usage
        self.data = torch.empty(numel, dtype=dtype, device=device, requires_grad=False)
        self._start = 0
        self.in_use_value = 0.0
        self.total_value = 0.0

    def reset(self) -> None:
        self._start = 0

    def is_in_use(self) -> bool:
        return self._start > 0

    def numel_in_use(self) -> int:
        return self._start

    def add(self, tensor: torch.Tensor) -> torch.Tensor:
        """Copies `tensor` into the buffer and returns the view that now holds it."""
        assert tensor.dtype == self.dtype, f"buffer {self.name} holds {self.dtype}, got {tensor.dtype}"
        out = self.get(tensor.shape)
        out.copy_(tensor)
        return out

    def get(self, shape) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        end = self._start + n
        assert end <= self.numel, f"not enough memory left in buffer {self.name}: {end} > {self.numel}"
        out = self.data[self._start:end].view(tuple(shape))
        self._start = end
        return out

    def get_data(self) -> torch.Tensor:
        if self.track_usage:
            self.in_use_value += float(self._start)
            self.total_value += float(self.numel)
        return self.data[: self._start]

    def usage(self) -> float:
        """Average fraction of the buffer that was in use over the get_data() calls so far."""
        assert self.track_usage, "usage tracking is off"
        return self.in_use_value / max(self.total_value, 1.0)


class RingMemBuffer:
    def __init__(self, name: str, num_buffers: int, numel: int, dtype: torch.dtype, track_usage: bool = False,
                 device=None):
        self.buffers = [MemoryBuffer(f"{name} {i}", numel, dtype, track_usage, device) for i in range(num_buffers)]
        self._index = -1

    def get_next_buffer(self) -> MemoryBuffer:
        self._index = (self._index + 1) % len(self.buffers)
        buf = self.buffers[self._index]
        assert not buf.is_in_use(), "buffer is already in use"
        return buf


def report_memory(name: str = "", get_list: bool = False):
    """'[name] memory (MB) | allocated | max allocated | reserved | max reserved' and optionally the four numbers."""
    mb = 1024.0 * 1024.0
    if torch.cuda.is_available():
        vals = [torch.cuda.memory_allocated() / mb, torch.cuda.max_memory_allocated() / mb,
                torch.cuda.memory_reserved() / mb, torch.cuda.max_memory_reserved() / mb]
    else:
        vals = [0.0, 0.0, 0.0, 0.0]
    text = (f"{name} memory (MB) | allocated: {vals[0]:.2f} | max allocated: {vals[1]:.2f} | "
            f"reserved: {vals[2]:.2f} | max reserved: {vals[3]:.2f}")
    return (text, vals) if get_list else text


def debug_mem_report(min_mb: float = 0.0) -> List[Tuple[str, tuple, int, float]]:
    """Live tensors found by the garbage collector, grouped by (device, dtype, shape): rows of
    (device / dtype, shape, count, total MB), largest first.  Views of one storage are counted once."""
    seen, groups = set(), {}
    for obj in gc.get_objects():
        try:
            if not torch.is_tensor(obj):
                continue
            key = obj.untyped_storage().data_ptr()
        except Exception:  # noqa: BLE001 - objects that fail on attribute access during a gc walk
            continue
        if key in seen:
            continue
        seen.add(key)
        g = (f"{obj.device} {obj.dtype}", tuple(obj.shape))
        cnt, mbs = groups.get(g, (0, 0.0))
        groups[g] = (cnt + 1, mbs + obj.untyped_storage().nbytes() / (1024.0 * 1024.0))
    rows = [(k[0], k[1], c, m) for k, (c, m) in groups.items() if m >= min_mb]
    rows.sort(key=lambda r: -r[3])
    return rows
