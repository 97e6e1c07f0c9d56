"""Host model of the epoch-flag protocol the in-kernel collectives use (csrc/comm_sm100.cu, gemm_ar_sm100.cu,
gemm_ag_sm100.cu), for reasoning about it and for testing its failure behaviour without a GPU.

Protocol: every (rank, slot) owns one 32-bit flag per peer.  A producer finishes its data, then stores the call's
epoch into the consumer's flag (release); the consumer polls its own flag until it is >= the epoch (acquire),
at most `limit` polls, and reports a timeout status instead of waiting for ever.  Epochs only grow, flags are never
reset: a flag left over from an earlier call can never satisfy a later wait, and a late flag of an earlier call is
harmless.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

OK, PEER_TIMEOUT = 0, 2


class FlagBoard:
    """flags[(owner, slot, peer)] as seen in the owner's memory."""

    def __init__(self, drop: Optional[Callable[[int, int, int, int], bool]] = None):
        self.flags: Dict[Tuple[int, int, int], int] = {}
        self.drop = drop          # drop(owner, slot, peer, epoch) -> True loses that store (fault injection)

    def post(self, owner: int, slot: int, peer: int, epoch: int) -> None:
        if self.drop is not None and self.drop(owner, slot, peer, epoch):
            return
        key = (owner, slot, peer)
        self.flags[key] = max(self.flags.get(key, 0), epoch)

    def wait(self, owner: int, slot: int, peer: int, epoch: int, limit: int = 1000,
             progress: Optional[Callable[[], None]] = None) -> int:
        for _ in range(limit):
            if self.flags.get((owner, slot, peer), 0) >= epoch:
                return OK
            if progress is not None:
                progress()        # lets a test interleave the producer
        return PEER_TIMEOUT


def barrier(board: FlagBoard, world: int, slot: int, epoch: int, limit: int = 1000) -> Dict[int, int]:
    """All-to-all arrival (block_barrier of comm_sm100.cu): returns the status of every rank."""
    for r in range(world):
        for p in range(world):
            board.post(p, slot, r, epoch)
    return {r: max(board.wait(r, slot, p, epoch, limit) for p in range(world)) for r in range(world)}
