"""Parallel state derived from a plan: stage rank ranges and per-op tensor / data parallel groups.

Rank layout (same as the reference, runtime/megatron/mpu/initialize.py:142-198): stages occupy
contiguous rank ranges in order; inside a stage of G GPUs an op with degrees (tp, dp), tp * dp = G,
arranges the stage's ranks as a [dp][tp] grid, i.e. the TP group of stage-local rank r is
{(r // tp) * tp + i} and its DP group is {(r % tp) + j * tp}.  Groups are created lazily and cached by
their rank tuple; every rank must request the same groups in the same order (`ensure_groups`).

One process drives one GPU.  With world size 1 no process group is needed at all.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass
class OpPlacement:
    tp: int
    dp: int
    tp_rank: int
    dp_rank: int
    tp_ranks: Tuple[int, ...]   # global ranks of my TP group
    dp_ranks: Tuple[int, ...]   # global ranks of my DP group


class ParallelState:
    def __init__(self, num_gpus_per_stage: Sequence[int], rank: int = 0, world_size: int = 1):
        self.num_gpus = list(num_gpus_per_stage)
        assert sum(self.num_gpus) == world_size, \
            f"plan needs {sum(self.num_gpus)} GPUs but the job has {world_size} ranks"
        self.rank, self.world_size = rank, world_size
        self.num_stages = len(self.num_gpus)
        self.stage_start = [sum(self.num_gpus[:i]) for i in range(self.num_stages)]
        self.stage = max(i for i in range(self.num_stages) if self.stage_start[i] <= rank)
        self.local_rank_in_stage = rank - self.stage_start[self.stage]
        self._groups: Dict[Tuple[int, ...], Optional[dist.ProcessGroup]] = {}

    # ---- topology ---------------------------------------------------------------------------
    def stage_ranks(self, stage: int) -> List[int]:
        s = self.stage_start[stage]
        return list(range(s, s + self.num_gpus[stage]))

    def same_node(self, ranks: Sequence[int]) -> bool:
        """True when `ranks` all run on one node, i.e. can map each other's memory over NVLink.  The launcher places
        LOCAL_WORLD_SIZE consecutive ranks on every node (torchrun's contract); without it the job is one node."""
        import os
        per_node = int(os.environ.get("LOCAL_WORLD_SIZE", "0")) or self.world_size
        return len({r // per_node for r in ranks}) <= 1

    def is_first_stage(self) -> bool:
        return self.stage == 0

    def is_last_stage(self) -> bool:
        return self.stage == self.num_stages - 1

    def placement(self, tp: int, dp: int, stage: Optional[int] = None, local_rank: Optional[int] = None) -> OpPlacement:
        stage = self.stage if stage is None else stage
        r = self.local_rank_in_stage if local_rank is None else local_rank
        g = self.num_gpus[stage]
        assert tp * dp == g, f"op degrees tp={tp} x dp={dp} do not match the stage's {g} GPUs"
        base = self.stage_start[stage]
        tp_rank, dp_rank = r % tp, r // tp
        tp_ranks = tuple(base + dp_rank * tp + i for i in range(tp))
        dp_ranks = tuple(base + tp_rank + j * tp for j in range(dp))
        return OpPlacement(tp, dp, tp_rank, dp_rank, tp_ranks, dp_ranks)

    # ---- process groups ---------------------------------------------------------------------
    def group(self, ranks: Sequence[int]):
        """Process group over `ranks` (None for a single rank).  Must have been created by ensure_groups."""
        ranks = tuple(ranks)
        if len(ranks) <= 1:
            return None
        if ranks not in self._groups:
            raise KeyError(f"process group {ranks} was not created by ensure_groups()")
        return self._groups[ranks]

    def ensure_groups(self, all_rank_sets: Sequence[Sequence[int]]) -> None:
        """Collective: every rank passes the same ordered list of rank sets; new ones are created."""
        for ranks in all_rank_sets:
            ranks = tuple(ranks)
            if len(ranks) <= 1 or ranks in self._groups:
                continue
            if len(ranks) == self.world_size:
                self._groups[ranks] = dist.group.WORLD
            else:
                self._groups[ranks] = dist.new_group(list(ranks))

    def all_op_groups(self, tp_dp_per_stage: Sequence[Sequence[Tuple[int, int]]]) -> List[Tuple[int, ...]]:
        """Every TP and DP group any op of any stage needs, in a deterministic order."""
        seen, out = set(), []
        for stage, pairs in enumerate(tp_dp_per_stage):
            for tp, dp in sorted(set(pairs)):
                for r in range(self.num_gpus[stage]):
                    pl = self.placement(tp, dp, stage, r)
                    for ranks in (pl.tp_ranks, pl.dp_ranks):
                        if len(ranks) > 1 and ranks not in seen:
                            seen.add(ranks)
                            out.append(ranks)
            ranks = tuple(self.stage_ranks(stage))
            if len(ranks) > 1 and ranks not in seen:
                seen.add(ranks)
                out.append(ranks)
        return out


def init_distributed(backend: Optional[str] = None) -> Tuple[int, int, int]:
    """Reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* from the environment (torchrun contract)."""
    import os
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, world, local
