"""Differentiable collectives over explicit process groups (the NCCL baseline path).

Forward / backward pairs follow the conjugate rule used by the reference
(runtime/megatron/mpu/mappings.py:30-145 for the Megatron f/g operators, :212-303 for the
resharding primitives): identity <-> all-reduce, split <-> all-gather, reduce-scatter <-> all-gather,
all-to-all <-> all-to-all with swapped dimensions.  A `group` of None means a single rank: every
function is then the identity, so single-GPU code pays nothing.

No function synchronises the host: collectives are enqueued on the current stream by
torch.distributed and ordered by the stream (the reference calls torch.cuda.synchronize() after
every resharding collective, runtime/megatron/mpu/mappings.py:168,184,196,207).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _size(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


def _rank(group) -> int:
    return 0 if group is None else dist.get_rank(group)


def all_reduce_(t, group):
    if _size(group) > 1:
        dist.all_reduce(t, group=group)
    return t


def _all_gather(t, dim, group):
    n = _size(group)
    if n == 1:
        return t
    t = t.contiguous()
    if dim == 0:
        out = torch.empty((n * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=group)
        return out
    parts = [torch.empty_like(t) for _ in range(n)]
    dist.all_gather(parts, t, group=group)
    return torch.cat(parts, dim=dim)


def _split(t, dim, group):
    n = _size(group)
    if n == 1:
        return t
    return t.chunk(n, dim=dim)[_rank(group)].contiguous()


def _reduce_scatter(t, dim, group):
    n = _size(group)
    if n == 1:
        return t
    if dim != 0:
        t = torch.cat(t.chunk(n, dim=dim), dim=0)
    t = t.contiguous()
    out = torch.empty((t.shape[0] // n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.reduce_scatter_tensor(out, t, group=group)
    return out


def _all_to_all(t, split_dim, cat_dim, group):
    """Splits `split_dim` across the group and concatenates the received pieces along `cat_dim`."""
    n = _size(group)
    if n == 1:
        return t
    ins = [p.contiguous() for p in t.chunk(n, dim=split_dim)]
    if dist.get_backend(group) == "gloo":
        # gloo has no all-to-all: every rank gathers all inputs and keeps the pieces addressed to it (CPU tests)
        everything = [torch.empty_like(t) for _ in range(n)]
        dist.all_gather(everything, t.contiguous(), group=group)
        outs = [e.chunk(n, dim=split_dim)[_rank(group)] for e in everything]
        return torch.cat(outs, dim=cat_dim)
    outs = [torch.empty_like(ins[0]) for _ in range(n)]
    dist.all_to_all(outs, ins, group=group)
    return torch.cat(outs, dim=cat_dim)


class CopyToGroup(torch.autograd.Function):
    """identity forward, all-reduce backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        return all_reduce_(g.clone() if _size(ctx.group) > 1 else g, ctx.group), None


class ReduceFromGroup(torch.autograd.Function):
    """all-reduce forward, identity backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        return all_reduce_(x.contiguous(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class GatherFromGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _all_gather(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        return _split(g, ctx.dim, ctx.group), None, None


class SplitToGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _split(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather(g, ctx.dim, ctx.group), None, None


class ReduceScatterToGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        return _reduce_scatter(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather(g, ctx.dim, ctx.group), None, None


class AllToAllInGroup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, split_dim, cat_dim, group):
        ctx.dims, ctx.group = (split_dim, cat_dim), group
        return _all_to_all(x, split_dim, cat_dim, group)

    @staticmethod
    def backward(ctx, g):
        s, c = ctx.dims
        return _all_to_all(g, c, s, ctx.group), None, None, None


def copy_to_group(x, group):
    return x if _size(group) == 1 else CopyToGroup.apply(x, group)


def reduce_from_group(x, group):
    return x if _size(group) == 1 else ReduceFromGroup.apply(x, group)


def gather_from_group(x, dim, group):
    return x if _size(group) == 1 else GatherFromGroup.apply(x, dim, group)


def split_to_group(x, dim, group):
    return x if _size(group) == 1 else SplitToGroup.apply(x, dim, group)


def reduce_scatter_to_group(x, dim, group):
    return x if _size(group) == 1 else ReduceScatterToGroup.apply(x, dim, group)


def all_to_all_in_group(x, split_dim, cat_dim, group):
    return x if _size(group) == 1 else AllToAllInGroup.apply(x, split_dim, cat_dim, group)
