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
        nflags = native.ext().comm_max_blocks() * self.world
        off = flag_off = 0
        if os.environ.get("SSB_CANARIES", "0") == "1":
            # guard words in front of and behind both buffers (parallel/guards.py); every rank does the same, so the
            # payloads start at the same offset of the symmetric allocations
            from .guards import REGISTRY, GuardedBuffer
            alloc = lambda n, dtype, device: symm.empty(n, dtype=dtype, device=device)      # noqa: E731
            data = REGISTRY.add(GuardedBuffer(numel, dtype, device, alloc=alloc, name=f"symmetric buffer of {numel}"))
            flg = REGISTRY.add(GuardedBuffer(nflags, torch.int32, device, alloc=alloc, name="symmetric flag table"))
            raw, self.tensor, off = data.raw, data.body, data.body_offset_bytes
            raw_flags, self.flags, flag_off = flg.raw, flg.body, flg.body_offset_bytes
        else:
            raw = self.tensor = symm.empty(numel, dtype=dtype, device=device)
            raw_flags = self.flags = symm.empty(nflags, dtype=torch.int32, device=device)
        self.tensor.zero_()
        self.flags.zero_()
        self.handle = symm.rendezvous(raw, self.group.group_name)
        self.flag_handle = symm.rendezvous(raw_flags, self.group.group_name)
        self.peer_ptrs = torch.tensor([p + off for p in self.handle.buffer_ptrs], dtype=torch.int64, device=device)
        self.flag_ptrs = torch.tensor([p + flag_off for p in self.flag_handle.buffer_ptrs], dtype=torch.int64, device=device)
        use_nvls = os.environ.get("SSB_DISABLE_MULTIMEM", "0") != "1"
        mc = 0
        if use_nvls:
            try:
                mc = int(self.handle.multicast_ptr or 0)
                mc = mc + off if mc else 0
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

    def _tables_at(self, offset: int):
        """Pointer tables (peer addresses, multicast address) of the sub-buffer that starts `offset` elements in."""
        if offset == 0:
            return self.peer_ptrs, self.multicast_ptr
        cache = self.__dict__.setdefault("_offset_tables", {})
        if offset not in cache:
            nbytes = offset * self.tensor.element_size()
            cache[offset] = (self.peer_ptrs + nbytes, self.multicast_ptr + nbytes if self.multicast_ptr else 0)
        return cache[offset]

    def allreduce_scale_(self, numel: Optional[int] = None, scale: float = 1.0, offset: int = 0) -> None:
        """In place on `self.tensor[offset:offset + numel]` (fp32): sum over the group's ranks, times `scale`."""
        from ..ops import native
        n = self.tensor.numel() - offset if numel is None else numel
        assert self.tensor.dtype == torch.float32 and n % 4 == 0 and offset % 4 == 0
        ptrs, mc = self._tables_at(offset)
        native.ext().allreduce_scale_f32(ptrs, mc, self.flag_ptrs, self.rank, self.world, n, scale, self.next_epoch())

    def slice_of(self, numel: int):
        """[lo, hi) of this rank's slice of the first `numel` elements, as the two kernels below deal them out."""
        from ..ops import native
        lo, hi = native.ext().comm_slice(numel, self.world, self.rank)
        return int(lo), int(hi)

    def reduce_scatter_scale_sumsq_(self, numel: int, scale: float, partials: torch.Tensor) -> None:
        """fp32: this rank's slice of `self.tensor[:numel]` becomes the sum over the ranks times `scale`, the rest of
        `self.tensor[:numel]` is cleared, `partials` receives per-block sums of squares of the reduced slice."""
        from ..ops import native
        assert self.tensor.dtype == torch.float32 and numel % 8 == 0
        native.ext().reduce_scatter_scale_sumsq_f32(self.peer_ptrs, self.multicast_ptr, self.flag_ptrs, self.rank,
                                                    self.world, numel, scale, self.next_epoch(), partials)

    def allgather_(self, numel: int) -> None:
        """16-bit buffer: every rank's slice of `self.tensor[:numel]` is copied into every other rank's buffer."""
        from ..ops import native
        assert self.tensor.element_size() == 2 and numel % 8 == 0
        native.ext().allgather_b16(self.peer_ptrs, self.multicast_ptr, self.flag_ptrs, self.rank, self.world, numel,
                                   self.next_epoch())


class FusedTPContext:
    """Symmetric scratch of one tensor-parallel group for the fused GEMM + all-reduce kernel
    (csrc/gemm_ar_sm100.cu): a bf16 buffer that receives the partial tiles this rank owns, two alternating result
    buffers that receive the final tiles of the other owners, and the flag table, each rendezvoused once;
    `linear_allreduce` launches the kernel.  All ranks of the group must issue the same sequence of calls
    (shapes included), which SPMD execution of one plan guarantees."""

    TILE_M, TILE_N = 128, 256

    def __init__(self, group, max_rows: int, max_cols: int, device):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.tp = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device
        tiles = -(-max_rows // self.TILE_M) * -(-max_cols // self.TILE_N)
        self.max_tiles = tiles
        self.capacity = (tiles + self.tp) * self.TILE_M * self.TILE_N     # buffers hold whole (padded) tiles
        name = self.group.group_name

        def table(t):
            h = symm.rendezvous(t, name)
            return h, torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=device)

        self.partial = symm.empty(self.capacity, dtype=torch.bfloat16, device=device)
        self.results = [symm.empty(self.capacity, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.flags = symm.empty(self.max_tiles * (self.tp * 4 + 4) + self.tp + 1, dtype=torch.int32, device=device)
        self.flags.zero_()
        _, self.partial_ptrs = table(self.partial)
        handles = [table(r) for r in self.results]
        self.result_ptrs = [h[1] for h in handles]
        _, self.flag_ptrs = table(self.flags)
        self.epoch = 0
        self.last_scatter_epoch = 0     # epoch of the last reduce-scatter call: later calls wait for its "consumed" flags
        torch.cuda.synchronize(device)
        dist.barrier(self.group)

    def fits(self, rows: int, cols: int) -> bool:
        return -(-rows // self.TILE_M) * -(-cols // self.TILE_N) <= self.max_tiles

    def linear_allreduce(self, x: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, bias=None, residual=None,
                         alpha: float = 1.0, dropout_p: float = 0.0, seed: int = 0, out=None) -> torch.Tensor:
        """sum over the group of (x_r . w_r^T) [+ bias, dropout, + residual] on every rank."""
        from ..ops import native
        M = x.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        assert self.fits(M, N), f"fused TP scratch too small for {M}x{N}"
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        self.epoch += 1
        par = self.epoch & 1
        native.ext().gemm_allreduce(x, w, b_mn, out, bias, residual, alpha, dropout_p, seed, self.partial_ptrs,
                                    self.result_ptrs[par], self.flag_ptrs, self.rank, self.tp, self.epoch,
                                    self.max_tiles, self.capacity, False, self.last_scatter_epoch)
        return out

    def linear_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, bias=None, residual=None,
                              alpha: float = 1.0, dropout_p: float = 0.0, seed: int = 0, out=None) -> torch.Tensor:
        """Rows [r M / tp, (r + 1) M / tp) of sum over the group of (x_r . w_r^T) [+ bias, dropout, + residual] on rank
        r: the GEMM -> reduce-scatter form of the same kernel (nothing travels back to the peers).  M / tp must be a
        multiple of 128.  `residual` and the result are this rank's [M / tp, N] rows."""
        from ..ops import native
        M = x.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        assert self.fits(M, N), f"fused TP scratch too small for {M}x{N}"
        assert M % (self.tp * self.TILE_M) == 0, "rows per rank must be a multiple of 128"
        if out is None:
            out = torch.empty((M // self.tp, N), dtype=torch.bfloat16, device=x.device)
        self.epoch += 1
        par = self.epoch & 1
        native.ext().gemm_allreduce(x, w, b_mn, out, bias, residual, alpha, dropout_p, seed, self.partial_ptrs,
                                    self.result_ptrs[par], self.flag_ptrs, self.rank, self.tp, self.epoch,
                                    self.max_tiles, self.capacity, True, self.last_scatter_epoch)
        self.last_scatter_epoch = self.epoch
        return out

    # ---- all-gather fused into the consuming GEMM (csrc/gemm_ag_sm100.cu) -------------------------------------
    def enable_allgather(self, max_rows_total: int, max_k: int) -> None:
        """Allocates (collectively, once) the two alternating gather buffers [rows, K] and their flag table."""
        import torch.distributed._symmetric_memory as symm
        name = self.group.group_name
        self.ag_capacity = int(max_rows_total) * int(max_k)
        self.ag_max_blocks = -(-int(max_rows_total) // self.TILE_M)
        self.ag_bufs = [symm.empty(self.ag_capacity, dtype=torch.bfloat16, device=self.device) for _ in range(2)]
        self.ag_flags = symm.empty(self.ag_max_blocks, dtype=torch.int32, device=self.device)
        self.ag_flags.zero_()
        self.ag_ptrs, self.ag_local = [], []
        for b in self.ag_bufs:
            h = symm.rendezvous(b, name)
            self.ag_ptrs.append(torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=self.device))
            self.ag_local.append(int(h.buffer_ptrs[self.rank]))
        h = symm.rendezvous(self.ag_flags, name)
        self.ag_flag_ptrs = torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=self.device)
        self.ag_epoch = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def ensure_allgather(self, rows_total: int, k: int) -> None:
        """Collective on first use (every rank of the group reaches it with the same arguments): makes the gather
        scratch large enough for [rows_total, k]."""
        if getattr(self, "ag_capacity", 0) < rows_total * k or getattr(self, "ag_max_blocks", 0) < -(-rows_total // self.TILE_M):
            self.enable_allgather(rows_total, k)

    def gathered_input(self, x_local: torch.Tensor) -> torch.Tensor:
        """The full [rows * tp, K] input of the LAST allgather_linear call, as a tensor of its own: the peers' rows out
        of this rank's gather scratch (every one of them has arrived when that kernel ends), this rank's rows from
        `x_local` (the kernel reads them in place and never copies them)."""
        rows, K = x_local.shape
        M = rows * self.tp
        full = self.ag_bufs[self.ag_epoch & 1][:M * K].view(M, K).clone()
        full[self.rank * rows:(self.rank + 1) * rows] = x_local
        return full

    def allgather_linear(self, x_local: torch.Tensor, w: torch.Tensor, *, bias=None, act: int = 0, preact_out=None,
                         out=None) -> torch.Tensor:
        """act(concat over the group of x_r . w^T + bias): rows of rank r land at [r * rows, (r + 1) * rows)."""
        from ..ops import native
        rows, K = x_local.shape
        M, N = rows * self.tp, w.shape[0]
        assert rows % self.TILE_M == 0 and K % 64 == 0, "rows per rank must be a multiple of 128, K of 64"
        assert M * K <= self.ag_capacity and M // self.TILE_M <= self.ag_max_blocks, "gather scratch too small"
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x_local.device)
        self.ag_epoch += 1
        par = self.ag_epoch & 1
        native.ext().allgather_gemm(x_local.contiguous(), w, out, bias, act, preact_out, self.ag_ptrs[par],
                                    self.ag_local[par], self.ag_flag_ptrs, self.rank, self.tp, self.ag_epoch,
                                    self.ag_max_blocks, self.ag_capacity)
        return out
