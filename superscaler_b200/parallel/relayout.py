"""Relayout engine: moves a logically global tensor between two sharded layouts, possibly held by two
different sets of ranks.

One mechanism serves both places where the reference moves activations between layouts:
  * pipeline stage boundaries, where the two stages may have different GPU counts and the tensor is
    re-chunked by the child's tp x dp (runtime/megatron/p2p_communication.py:84-201,203-337);
  * inside a stage, between consecutive ops whose (tp, dp, algo) differ
    (`tensor_adapter`, runtime/megatron/mpu/mappings.py:382-468).

A tensor's layout says how dim 0 (rows: tokens / samples) and dim 1 (features / heads) are held:
  row "split": dim 0 is cut into dp contiguous blocks, block i on data-parallel rank i; "rep": every rank has all rows
  col "split": dim 1 is cut over the tp ranks, separately inside each of `groups` equal column groups
               (3 for a fused [Q|K|V] matrix); "rep": every tensor-parallel rank holds all columns.
Ranks of a side are contiguous and arranged [dp][tp] (local rank = dp_rank * tp + tp_rank).

The transfer plan is a pure function of (sides, layouts, global shape), computed identically on every
rank.  Forward: every destination rank fetches each piece of its region from exactly one owner (replicas
are spread over the requesters).  Backward is the same plan with the sides swapped; gradients of replicas
along a split-capable axis are identical, so one representative is read, while row-"rep" tensors
(parameters riding with the activations, e.g. a deferred bias) differ per data-parallel rank and are
averaged over them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Layout:
    row: str = "split"
    col: str = "rep"
    groups: int = 1


@dataclass(frozen=True)
class Side:
    first_rank: int
    tp: int
    dp: int

    @property
    def size(self) -> int:
        return self.tp * self.dp

    def rank(self, dp_rank: int, tp_rank: int) -> int:
        return self.first_rank + dp_rank * self.tp + tp_rank

    def coords(self, rank: int) -> Tuple[int, int]:
        r = rank - self.first_rank
        return r // self.tp, r % self.tp

    def contains(self, rank: int) -> bool:
        return self.first_rank <= rank < self.first_rank + self.size


@dataclass(frozen=True)
class Piece:
    r0: int
    r1: int          # global rows [r0, r1)
    group: int
    c0: int
    c1: int          # columns inside the group [c0, c1)


@dataclass
class Message:
    src: int
    dst: int
    pieces: List[Piece]
    scale: float = 1.0


def _row_blocks(side: Side, lay: Layout, rows: int, dp_rank: int) -> Tuple[int, int]:
    if lay.row == "split":
        per = rows // side.dp
        return dp_rank * per, (dp_rank + 1) * per
    return 0, rows


def _col_block(side: Side, lay: Layout, gcols: int, tp_rank: int) -> Tuple[int, int]:
    if lay.col == "split":
        per = gcols // side.tp
        return tp_rank * per, (tp_rank + 1) * per
    return 0, gcols


def local_shape(side: Side, lay: Layout, gshape: Sequence[int]) -> Tuple[int, ...]:
    rows = gshape[0] // side.dp if lay.row == "split" else gshape[0]
    if len(gshape) == 1:
        return (rows,)
    cols = gshape[1] // side.tp if lay.col == "split" else gshape[1]
    return (rows, cols) + tuple(gshape[2:])


def global_shape(side: Side, lay: Layout, lshape: Sequence[int]) -> Tuple[int, ...]:
    rows = lshape[0] * side.dp if lay.row == "split" else lshape[0]
    if len(lshape) == 1:
        return (rows,)
    cols = lshape[1] * side.tp if lay.col == "split" else lshape[1]
    return (rows, cols) + tuple(lshape[2:])


def plan_transfer(src: Side, src_lay: Layout, dst: Side, dst_lay: Layout, gshape: Sequence[int],
                  sum_row_replicas: bool = False) -> List[Message]:
    """Messages that give every rank of `dst` its region under `dst_lay` from the owners under `src_lay`.

    sum_row_replicas marks the gradient direction: row-replicated tensors add the contributions of ALL
    data-parallel ranks of `src`, each scaled by 1 / src.dp; row-split tensors are scaled by dst.dp / src.dp."""
    rows = gshape[0]
    cols = gshape[1] if len(gshape) > 1 else 1
    groups = src_lay.groups
    assert dst_lay.groups == groups and cols % groups == 0
    gcols = cols // groups
    msgs: Dict[Tuple[int, int], Message] = {}
    for ddp in range(dst.dp):
        for dtp in range(dst.tp):
            d_rank = dst.rank(ddp, dtp)
            r0, r1 = _row_blocks(dst, dst_lay, rows, ddp)
            c0, c1 = _col_block(dst, dst_lay, gcols, dtp)
            # row owners
            if src_lay.row == "split":
                per = rows // src.dp
                row_src = [(k, max(r0, k * per), min(r1, (k + 1) * per)) for k in range(src.dp)
                           if max(r0, k * per) < min(r1, (k + 1) * per)]
                # Every rank differentiates the MEAN loss of its own rows.  Where the data-parallel degree
                # changes, the gradient is rescaled so that the usual 1/dp averaging of the parameter
                # gradients on the receiving side still yields the gradient of the global mean.
                scale = (dst.dp / src.dp) if sum_row_replicas else 1.0
            elif sum_row_replicas:
                row_src = [(k, r0, r1) for k in range(src.dp)]
                scale = 1.0 / src.dp
            else:
                row_src = [(ddp % src.dp, r0, r1)]
                scale = 1.0
            # column owners
            if src_lay.col == "split":
                per = gcols // src.tp
                col_src = [(k, max(c0, k * per), min(c1, (k + 1) * per)) for k in range(src.tp)
                           if max(c0, k * per) < min(c1, (k + 1) * per)]
            else:
                col_src = [(dtp % src.tp, c0, c1)]
            for sdp, a0, a1 in row_src:
                for stp, b0, b1 in col_src:
                    s_rank = src.rank(sdp, stp)
                    m = msgs.setdefault((s_rank, d_rank), Message(s_rank, d_rank, [], scale))
                    for g in range(groups):
                        m.pieces.append(Piece(a0, a1, g, b0, b1))
    return [msgs[k] for k in sorted(msgs)]


def _slice_of(side: Side, lay: Layout, rank: int, p: Piece, rows: int, gcols: int):
    """Local (row slice, col slice) of piece `p` inside the tensor held by `rank`."""
    dpr, tpr = side.coords(rank)
    rb0, _ = _row_blocks(side, lay, rows, dpr)
    cb0, cb1 = _col_block(side, lay, gcols, tpr)
    width = cb1 - cb0
    c_lo = p.group * width + (p.c0 - cb0)
    return slice(p.r0 - rb0, p.r1 - rb0), slice(c_lo, c_lo + (p.c1 - p.c0))


def _pack(t: torch.Tensor, side: Side, lay: Layout, rank: int, msg: Message, gshape) -> torch.Tensor:
    rows = gshape[0]
    if t.dim() == 1:
        parts = [t[p.r0 - _row_blocks(side, lay, rows, side.coords(rank)[0])[0]:
                   p.r1 - _row_blocks(side, lay, rows, side.coords(rank)[0])[0]].reshape(-1) for p in msg.pieces]
        return torch.cat(parts) if len(parts) > 1 else parts[0].contiguous()
    gcols = gshape[1] // lay.groups
    parts = []
    for p in msg.pieces:
        rs, cs = _slice_of(side, lay, rank, p, rows, gcols)
        parts.append(t[rs, cs].reshape(-1))
    return torch.cat(parts) if len(parts) > 1 else parts[0].contiguous()


def _unpack(buf: torch.Tensor, out: torch.Tensor, side: Side, lay: Layout, rank: int, msg: Message, gshape,
            accumulate: bool) -> None:
    rows = gshape[0]
    off = 0
    rest = 1
    for d in gshape[2:]:
        rest *= d
    if out.dim() == 1:
        rb0 = _row_blocks(side, lay, rows, side.coords(rank)[0])[0]
        for p in msg.pieces:
            n = p.r1 - p.r0
            piece = buf[off:off + n] * msg.scale if msg.scale != 1.0 else buf[off:off + n]
            if accumulate:
                out[p.r0 - rb0:p.r1 - rb0] += piece
            else:
                out[p.r0 - rb0:p.r1 - rb0] = piece
            off += n
        return
    gcols = gshape[1] // lay.groups
    for p in msg.pieces:
        rs, cs = _slice_of(side, lay, rank, p, rows, gcols)
        n = (p.r1 - p.r0) * (p.c1 - p.c0) * rest
        piece = buf[off:off + n].view((p.r1 - p.r0, p.c1 - p.c0) + tuple(gshape[2:]))
        if msg.scale != 1.0:
            piece = piece * msg.scale
        if accumulate:
            out[rs, cs] += piece
        else:
            out[rs, cs] = piece
        off += n


def _msg_numel(msg: Message, gshape) -> int:
    rest = 1
    for d in gshape[2:]:
        rest *= d
    if len(gshape) == 1:
        return sum(p.r1 - p.r0 for p in msg.pieces)
    return sum((p.r1 - p.r0) * (p.c1 - p.c0) for p in msg.pieces) * rest


class Transfer:
    """A prepared transfer of ONE tensor key between two sides; `post()` enqueues the sends / receives of this
    rank and returns a completion callback that yields the assembled local tensor (or None for pure senders)."""

    def __init__(self, my_rank: int, src: Side, src_lay: Layout, dst: Side, dst_lay: Layout, gshape, dtype, device,
                 sum_row_replicas: bool = False):
        self.rank, self.src, self.dst = my_rank, src, dst
        self.src_lay, self.dst_lay, self.gshape = src_lay, dst_lay, tuple(gshape)
        self.dtype, self.device = dtype, device
        msgs = plan_transfer(src, src_lay, dst, dst_lay, gshape, sum_row_replicas)
        self.sends = [m for m in msgs if m.src == my_rank]
        self.recvs = [m for m in msgs if m.dst == my_rank]
        self.accumulate = sum_row_replicas and src_lay.row == "rep" and src.dp > 1
        self.is_receiver = dst.contains(my_rank)

    def prepare(self, t: Optional[torch.Tensor]):
        """Returns (P2POps of this rank, assemble()).  The caller batches the ops of several transfers into one
        group call, waits for the requests and then calls assemble()."""
        ops, recv_bufs, local = [], [], []
        for m in self.sends:
            buf = _pack(t, self.src, self.src_lay, self.rank, m, self.gshape)
            if m.dst == self.rank:
                local.append((m, buf))
            else:
                ops.append(dist.P2POp(dist.isend, buf, m.dst))
        for m in self.recvs:
            if m.src == self.rank:
                continue
            buf = torch.empty(_msg_numel(m, self.gshape), dtype=self.dtype, device=self.device)
            recv_bufs.append((m, buf))
            ops.append(dist.P2POp(dist.irecv, buf, m.src))

        def assemble() -> Optional[torch.Tensor]:
            if not self.is_receiver:
                return None
            shape = local_shape(self.dst, self.dst_lay, self.gshape)
            out = (torch.zeros if self.accumulate else torch.empty)(shape, dtype=self.dtype, device=self.device)
            for m, buf in local + recv_bufs:
                _unpack(buf, out, self.dst, self.dst_lay, self.rank, m, self.gshape, self.accumulate)
            return out

        return ops, assemble

    def post(self, t: Optional[torch.Tensor]):
        ops, assemble = self.prepare(t)
        reqs = dist.batch_isend_irecv(ops) if ops else []

        def finish() -> Optional[torch.Tensor]:
            for r in reqs:
                r.wait()
            return assemble()

        return finish


class RelayoutFn(torch.autograd.Function):
    """Differentiable in-stage relayout (both sides are the same ranks)."""

    @staticmethod
    def forward(ctx, t, my_rank, src, src_lay, dst, dst_lay):
        g = global_shape(src, src_lay, t.shape)
        ctx.info = (my_rank, src, src_lay, dst, dst_lay, g, t.dtype, t.device)
        return Transfer(my_rank, src, src_lay, dst, dst_lay, g, t.dtype, t.device).post(t.contiguous())()

    @staticmethod
    def backward(ctx, grad):
        my_rank, src, src_lay, dst, dst_lay, g, dtype, device = ctx.info
        back = Transfer(my_rank, dst, dst_lay, src, src_lay, g, dtype, device, sum_row_replicas=True)
        return back.post(grad.contiguous())(), None, None, None, None, None


def relayout(t, my_rank: int, src: Side, src_lay: Layout, dst: Side, dst_lay: Layout):
    if src == dst and src_lay == dst_lay:
        return t
    return RelayoutFn.apply(t, my_rank, src, src_lay, dst, dst_lay)
