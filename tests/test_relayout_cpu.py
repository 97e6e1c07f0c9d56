"""Relayout engine: transfer plans and data movement between sharded layouts (gloo ranks on CPU)."""
import itertools

import pytest
import torch

from superscaler_b200.parallel.relayout import (Layout, Side, Transfer, global_shape, local_shape, plan_transfer,
                                                relayout)

from dist_utils import run_ranks


def _local(G, side, lay, rank):
    """Ground truth: the part of global tensor G that `rank` holds under `lay`."""
    dpr, tpr = side.coords(rank)
    t = G
    if lay.row == "split":
        t = t.chunk(side.dp, 0)[dpr]
    if lay.col == "split" and t.dim() > 1:
        parts = [g.chunk(side.tp, 1)[tpr] for g in t.chunk(lay.groups, 1)]
        t = torch.cat(parts, 1)
    return t.contiguous()


LAYOUTS = [Layout("split", "rep"), Layout("split", "split"), Layout("split", "split", 3), Layout("rep", "rep"),
           Layout("rep", "split")]


def test_plan_covers_every_destination_exactly_once():
    for (stp, sdp), (dtp, ddp) in itertools.product([(1, 1), (2, 1), (1, 2), (2, 2), (4, 1), (1, 4)], repeat=2):
        for sl, dl in itertools.product(LAYOUTS, repeat=2):
            if sl.groups != dl.groups or sl.row != dl.row:
                continue
            src, dst = Side(0, stp, sdp), Side(stp * sdp, dtp, ddp)
            g = (8, 24)
            msgs = plan_transfer(src, sl, dst, dl, g)
            for r in range(dst.first_rank, dst.first_rank + dst.size):
                want = local_shape(dst, dl, g)
                got = sum((p.r1 - p.r0) * (p.c1 - p.c0) for m in msgs if m.dst == r for p in m.pieces)
                assert got == want[0] * want[1], (src, sl, dst, dl, r)


def _fwd_worker(rank, world, case):
    (stp, sdp), (dtp, ddp), sl, dl, same = case
    src = Side(0, stp, sdp)
    dst = Side(0 if same else src.size, dtp, ddp)
    torch.manual_seed(0)
    G = torch.randn(8, 24, 2)
    t = _local(G, src, sl, rank) if src.contains(rank) else None
    tr = Transfer(rank, src, sl, dst, dl, G.shape, G.dtype, "cpu")
    out = tr.post(t)()
    if dst.contains(rank):
        assert torch.equal(out, _local(G, dst, dl, rank)), (rank, case)
    else:
        assert out is None


@pytest.mark.parametrize("case", [
    ((2, 1), (1, 2), Layout("split", "rep"), Layout("split", "rep"), False),
    ((1, 2), (2, 1), Layout("split", "split", 3), Layout("split", "split", 3), False),
    ((2, 1), (2, 1), Layout("split", "rep"), Layout("split", "split"), True),      # replicated -> split (slice)
    ((2, 2), (2, 2), Layout("split", "split"), Layout("split", "rep"), True),      # split -> replicated (gather)
    ((4, 1), (1, 4), Layout("split", "split"), Layout("split", "split"), True),    # tp4 -> dp4 (all-to-all)
    ((1, 4), (2, 2), Layout("rep", "split"), Layout("rep", "split"), True),
    ((1, 1), (1, 4), Layout("split", "rep"), Layout("split", "rep"), False),
])
def test_forward_moves_the_right_data(case):
    (stp, sdp), (dtp, ddp), _, _, same = case
    world = max(stp * sdp, dtp * ddp) if same else stp * sdp + dtp * ddp
    run_ranks(_fwd_worker, world, case)


def _grad_worker(rank, world):
    # tp2 replicated -> dp2 split rows (and back): y = relayout(x); loss = sum(y * w)
    src, dst = Side(0, 2, 1), Side(0, 1, 2)
    torch.manual_seed(0)
    G = torch.randn(8, 6)
    W = torch.randn(8, 6)
    x = _local(G, src, Layout("split", "rep"), rank).clone().requires_grad_(True)
    y = relayout(x, rank, src, Layout("split", "rep"), dst, Layout("split", "rep"))
    (y * _local(W, dst, Layout("split", "rep"), rank)).sum().backward()
    # every replica receives the full gradient, scaled by dp_src / dp_dst = 1/2 (each destination rank
    # differentiates the mean over HALF of the rows)
    assert torch.allclose(x.grad, 0.5 * W)
    # column split over tp2 <-> replicated: conjugate pair gather / slice
    x2 = _local(G, src, Layout("split", "split"), rank).clone().requires_grad_(True)
    y2 = relayout(x2, rank, src, Layout("split", "split"), src, Layout("split", "rep"))
    assert torch.equal(y2, G)
    (y2 * W).sum().backward()
    assert torch.allclose(x2.grad, _local(W, src, Layout("split", "split"), rank))
    # a parameter-like tensor replicated over dp2: gradient is the mean over the data-parallel ranks
    b = torch.ones(6, requires_grad=True)
    dsrc, ddst = Side(0, 1, 2), Side(0, 1, 2)
    yb = relayout(b * 1.0, rank, dsrc, Layout("rep", "rep"), ddst, Layout("rep", "rep"))
    assert yb is not None


def test_backward_is_the_conjugate_transfer():
    run_ranks(_grad_worker, 2)


def _bcast_worker(rank, world):
    import torch
    import torch.distributed as dist
    from superscaler_b200.parallel.data import broadcast_batch
    group = dist.new_group([1, 2])
    other = dist.new_group([0, 3])
    keys = ["ids", "labels", "mask"]
    src = {"ids": torch.arange(12).view(3, 4), "labels": torch.arange(12).view(3, 4) + 1,
           "mask": torch.ones(3, 4, 2, dtype=torch.int64)}
    if rank in (1, 2):
        got = broadcast_batch(keys, src if rank == 1 else None, torch.int64, 1, group)
    else:
        got = broadcast_batch(keys, {k: v * 10 for k, v in src.items()} if rank == 3 else None, torch.int64, 3, other)
    scale = 1 if rank in (1, 2) else 10
    for k in keys:
        assert got[k].shape == src[k].shape and (got[k] == src[k] * scale).all(), (rank, k)


def test_broadcast_batch_inside_sub_groups():
    from dist_utils import run_ranks
    run_ranks(_bcast_worker, 4)


def test_pack_and_unpack_move_the_right_elements_for_every_layout_pair():
    """The whole forward data path (plan, packing on the owners, unpacking on the requesters) in one process, for
    every pair of sides with tp, dp in {1, 2, 4, 8} (same ranks or disjoint), every pair of layouts, 2-D and 3-D
    tensors: each destination rank must end up with exactly its region of the global tensor."""
    from superscaler_b200.parallel.relayout import _msg_numel, _pack, _unpack
    torch.manual_seed(0)
    shapes = [(16, 48), (16, 48, 3)]
    degrees = [(1, 1), (2, 1), (1, 2), (2, 2), (4, 1), (1, 4), (4, 2), (2, 4), (8, 1), (1, 8)]
    checked = 0
    for gshape in shapes:
        G = torch.randn(gshape)
        for (stp, sdp), (dtp, ddp) in itertools.product(degrees, repeat=2):
            for same in (True, False):
                src = Side(0, stp, sdp)
                dst = Side(0 if same else src.size, dtp, ddp)
                for sl, dl in itertools.product(LAYOUTS, repeat=2):
                    if sl.groups != dl.groups:
                        continue
                    held = {r: _local(G, src, sl, r) for r in range(src.first_rank, src.first_rank + src.size)}
                    outs = {r: torch.full(local_shape(dst, dl, gshape), float("nan"))
                            for r in range(dst.first_rank, dst.first_rank + dst.size)}
                    for m in plan_transfer(src, sl, dst, dl, gshape):
                        buf = _pack(held[m.src], src, sl, m.src, m, gshape)
                        assert buf.numel() == _msg_numel(m, gshape)
                        _unpack(buf, outs[m.dst], dst, dl, m.dst, m, gshape, False)
                    for r, out in outs.items():
                        assert torch.equal(out, _local(G, dst, dl, r)), (gshape, src, sl, dst, dl, r)
                        checked += 1
    assert checked > 10000
