"""Symmetric (peer-mapped) device buffers for the in-kernel collectives.

Allocation, handle exchange and the NVLS multicast mapping are delegated to
torch.distributed._symmetric_memory (plumbing); the kernels that move and reduce data through the mapped
peer / multicast addresses are this framework's own (csrc/comm_sm100.cu).  A `SymmetricBuffer` carries, on the
device, the table of every rank's address of the same buffer plus a zero-initialised flag buffer for the
epoch protocol, and hands out epochs (two per collective call) in lock-step on all ranks.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, group, device):
        import torch.distributed._symmetric_memory as symm
        from ..ops import native
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm.rendezvous(self.tensor, self.group.group_name)
        nflags = native.ext().comm_max_blocks() * self.world
        self.flags = symm.empty(nflags, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flag_handle = symm.rendezvous(self.flags, self.group.group_name)
        self.peer_ptrs = torch.tensor(list(self.handle.buffer_ptrs), dtype=torch.int64, device=device)
        self.flag_ptrs = torch.tensor(list(self.flag_handle.buffer_ptrs), dtype=torch.int64, device=device)
        use_nvls = os.environ.get("SSB_DISABLE_MULTIMEM", "0") != "1"
        mc = 0
        if use_nvls:
            try:
                mc = int(self.handle.multicast_ptr or 0)
            except Exception:  # noqa: BLE001 - no multicast support on this fabric
                mc = 0
        self.multicast_ptr = mc
        self._epoch = 1
        torch.cuda.synchronize(device)
        dist.barrier(self.group)

    def next_epoch(self) -> int:
        e = self._epoch
        self._epoch += 2
        return e

    def allreduce_scale_(self, numel: Optional[int] = None, scale: float = 1.0) -> None:
        """In place on `self.tensor[:numel]` (fp32): sum over the group's ranks, times `scale`."""
        from ..ops import native
        n = self.tensor.numel() if numel is None else numel
        assert self.tensor.dtype == torch.float32 and n % 4 == 0
        native.ext().allreduce_scale_f32(self.peer_ptrs, self.multicast_ptr, self.flag_ptrs, self.rank, self.world, n,
                                         scale, self.next_epoch())
