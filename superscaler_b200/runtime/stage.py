"""A pipeline stage: the ops [start, end) of the flat op list, their parameters, op fusion and per-op
recompute.

Counterpart of the reference's FlexPipeModel (runtime/megatron/model/flex_model.py:361-609): consecutive ops
whose plan says recompute = 1 form a checkpointed segment, with forced breaks before every
`*-1st-layernorm` and `*-conv1` (flex_model.py:564-588).  A checkpointed segment stores only its input
tensors and the dropout seed counter; backward replays it with gradients enabled.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Sequence

import torch

from ..models.base import Env, Op, OpInfo
from ..ops import functional as F
from ..parallel.relayout import Layout, Side, relayout


class _CheckpointFn(torch.autograd.Function):
    """Recompute-in-backward for a run of ops operating on a dict of named tensors.  The dropout seed counter
    is saved before the segment and replayed for the recomputation (the role of CheckpointFunction's RNG
    bookkeeping, runtime/megatron/mpu/random.py:246-326)."""

    @staticmethod
    def forward(ctx, run, in_keys, holder, split_groups, *tensors):
        ctx.run, ctx.in_keys = run, in_keys
        ctx.seed_state = F.seed_state().get_state()
        # an input every rank of a tensor-parallel group holds in full is kept as this rank's 1 / tp share and
        # gathered again for the replay (--distribute-checkpointed-activations of the reference,
        # runtime/megatron/mpu/random.py:262-276,291-294)
        kept, ctx.shares = [], []
        for t, g in zip(tensors, split_groups):
            if g is None:
                kept.append(t)
                ctx.shares.append(None)
                continue
            n, r = torch.distributed.get_world_size(g), torch.distributed.get_rank(g)
            flat = t.detach().reshape(-1)
            share = flat.numel() // n
            kept.append(flat[r * share:(r + 1) * share].clone())
            ctx.shares.append((g, n, t.shape))
        ctx.save_for_backward(*kept)
        ctx.req = [t.requires_grad for t in tensors]
        with torch.no_grad():
            st = dict(zip(in_keys, tensors))
            run(st)
        out_keys = [k for k, v in st.items() if isinstance(v, torch.Tensor)]
        holder["out_keys"] = out_keys
        ctx.out_keys = out_keys
        outs = tuple(st[k] for k in out_keys)
        # Inputs passed through unchanged must not be returned as the same tensor object, and neither may a
        # parameter an op hands on (the deferred bias of a projection whose dropout + add lies behind the segment's
        # end): autograd would make the returned object an output of this node, so the PARAMETER itself would get
        # this node as its grad_fn and the replay in backward would recurse into it.  Under no_grad only such
        # leaves can require grad; they are returned as views.
        ids_in = {id(t) for t in tensors}
        return tuple(o.view_as(o) if (id(o) in ids_in or o.requires_grad) else o for o in outs)

    @staticmethod
    def backward(ctx, *grads):
        tensors = list(ctx.saved_tensors)
        for i, info in enumerate(ctx.shares):
            if info is not None:
                g, n, shape = info
                whole = torch.empty(n * tensors[i].numel(), dtype=tensors[i].dtype, device=tensors[i].device)
                torch.distributed.all_gather_into_tensor(whole, tensors[i], group=g)
                tensors[i] = whole.view(shape)
        ins = []
        for t, r in zip(tensors, ctx.req):
            d = t.detach()
            d.requires_grad_(r and t.is_floating_point())
            ins.append(d)
        saved = F.seed_state().get_state()
        F.seed_state().set_state(ctx.seed_state)
        with torch.enable_grad():
            st = dict(zip(ctx.in_keys, ins))
            ctx.run(st)
        F.seed_state().set_state(saved)
        outs, gs = [], []
        for k, g in zip(ctx.out_keys, grads):
            o = st[k]
            if g is not None and isinstance(o, torch.Tensor) and o.requires_grad:
                outs.append(o)
                gs.append(g)
        if outs:
            torch.autograd.backward(outs, gs)
        return (None, None, None, None) + tuple(i.grad if i.requires_grad else None for i in ins)


def _same_layout(side_a: Side, lay_a: Layout, side_b: Side, lay_b: Layout) -> bool:
    """True when no data has to move: equal sides and layouts that only differ along an undivided axis."""
    if side_a != side_b:
        return False
    if lay_a.row != lay_b.row and side_a.dp > 1:
        return False
    if side_a.tp > 1 and (lay_a.col != lay_b.col or (lay_a.col == "split" and lay_a.groups != lay_b.groups)):
        return False
    return True


def _rows_gather_in_gemm(op: Op, t: torch.Tensor, cur_side: Side, cur_lay: Layout, side: Side) -> bool:
    """True when `t` holds this rank's share of rows dealt out over exactly the ranks of the op's tensor-parallel
    group (previous op: tp 1, dp = this op's tp; this op: dp 1) and the op can take them as they are: the K4 / K5
    path.  SSB_FUSED_GATHER=0 keeps the relayout engine (NCCL) for comparison."""
    import os
    if os.environ.get("SSB_FUSED_GATHER", "1") == "0" or not getattr(op, "accepts_dealt_out_rows", lambda: False)():
        return False
    if not (cur_side.first_rank == side.first_rank and cur_side.tp == 1 and side.dp == 1 and cur_side.dp == side.tp
            and side.tp > 1 and cur_lay.row == "split"):
        return False
    return F.can_gather_in_gemm(t, op.tpctx())


# Debugging: every entry is called as hook(op, state) right after an op's forward (the reference's post_forward_hook
# under DEBUG_OUTPUT, runtime/megatron/model/flex_model.py:245-247).  Empty in normal runs.
AFTER_OP_HOOKS: List[Callable] = []


def run_op(op: Op, st: Dict[str, torch.Tensor]) -> None:
    """Brings every tensor the op reads to the layout it requires under the op's own (tp, dp) -- the in-stage
    resharding of the reference's pre_forward_tensor_adapter_hook (flex_model.py:250-300) -- then runs it."""
    meta = st.get("_meta")
    if meta is None:
        op.forward(st)
        for hook in AFTER_OP_HOOKS:
            hook(op, st)
        return
    ps = op.env.pstate
    side = Side(ps.stage_start[ps.stage], op.info.tp, op.info.dp)
    if side.size > 1:
        req = op.required()
        for k in op.reads:
            t = st.get(k)
            if k in req and k in meta and isinstance(t, torch.Tensor):
                cur_side, cur_lay = meta[k]
                want = req[k]
                if cur_lay.groups != want.groups:
                    want = Layout(want.row, want.col, cur_lay.groups)
                if not _same_layout(cur_side, cur_lay, side, want):
                    if k == "x" and _rows_gather_in_gemm(op, t, cur_side, cur_lay, side):
                        # dp -> tp: the consumer is a column-parallel GEMM that gathers the rows itself, inside its
                        # kernel (and reduce-scatters the input gradient in its backward); nothing moves here
                        st["_x_rows_dealt_out"] = True
                        meta[k] = (side, want)
                        continue
                    one_d = t.dim() == 1
                    moved = relayout(t.unsqueeze(0) if one_d else t, ps.rank, cur_side, cur_lay, side, want)
                    st[k] = moved.squeeze(0) if one_d else moved
                meta[k] = (side, want)
    op.forward(st)
    for k, lay in op.produced().items():
        if k in st:
            meta[k] = (side, lay)
    for hook in AFTER_OP_HOOKS:
        hook(op, st)


class Segment:
    def __init__(self, ops: List[Op], recompute: bool):
        self.ops, self.recompute = ops, recompute

    def _shared_inputs(self, st, in_keys, meta_in) -> list:
        """Per input: the tensor-parallel group whose ranks all hold that tensor in full (so each may keep a share of
        it for the replay), or None.  Only with `Env.distribute_saved_activations`."""
        first = self.ops[0]
        env = first.env
        none = [None] * len(in_keys)
        if not getattr(env, "distribute_saved_activations", False) or meta_in is None or first.pl.tp == 1:
            return none
        ps = env.pstate
        here = Side(ps.stage_start[ps.stage], first.info.tp, first.info.dp)
        out = []
        for k in in_keys:
            t, m = st[k], meta_in.get(k)
            whole = (m is not None and m[0] == here and m[1].col == "rep" and t.is_floating_point() and t.dim() >= 2
                     and t.numel() % first.pl.tp == 0)
            out.append(first.tp_group if whole else None)
        return out

    def _run(self, st):
        for op in self.ops:
            run_op(op, st)

    def forward(self, st: Dict[str, torch.Tensor]) -> None:
        if not self.recompute or not torch.is_grad_enabled():
            self._run(st)
            return
        in_keys = [k for k, v in st.items() if isinstance(v, torch.Tensor)]
        extras = {k: v for k, v in st.items() if not isinstance(v, torch.Tensor) and k != "_meta"}
        meta_in = dict(st["_meta"]) if "_meta" in st else None
        meta_out: dict = {}

        def run(inner):
            inner.update(extras)  # plain Python values (scales, flags) are visible inside the segment too
            if meta_in is not None:
                inner["_meta"] = dict(meta_in)  # the replay starts from the same layouts as the first run
            self._run(inner)
            if meta_in is not None:
                meta_out.clear()
                meta_out.update(inner["_meta"])

        holder: dict = {}
        outs = _CheckpointFn.apply(run, in_keys, holder, self._shared_inputs(st, in_keys, meta_in),
                                   *[st[k] for k in in_keys])
        for k in in_keys:
            st.pop(k)
        for k, v in zip(holder["out_keys"], outs):
            st[k] = v
        if meta_in is not None:
            st["_meta"] = dict(meta_out)


def split_segments(ops: List[Op]) -> List[Segment]:
    """Maximal runs of equal recompute flag; a recomputed run is cut before each layer's first op."""
    segs: List[Segment] = []
    cur: List[Op] = []
    cur_flag = None
    for op in ops:
        flag = bool(op.info.recompute)
        name = op.info.name
        new_layer = name.endswith("1st-layernorm") or name.endswith("-conv1")
        if cur and (flag != cur_flag or (flag and new_layer)):
            segs.append(Segment(cur, cur_flag))
            cur = []
        cur.append(op)
        cur_flag = flag
    if cur:
        segs.append(Segment(cur, cur_flag))
    return segs


class Stage:
    """Ops + parameters of this rank's pipeline stage.  With interleaving a stage owns several model chunks
    (non-adjacent slices of the op list); all chunks share one parameter store and one optimizer launch."""

    def __init__(self, infos, env: Env, build_op: Callable[[OpInfo, Env], Op], fuse=None):
        self.env = env
        chunks: List[Sequence[OpInfo]] = list(infos) if infos and isinstance(infos[0], (list, tuple)) else [infos]
        env.stage_ops = [i for c in chunks for i in c]
        self.raw_chunks: List[List[Op]] = [[build_op(i, env) for i in c] for c in chunks]
        self.raw_ops: List[Op] = [op for c in self.raw_chunks for op in c]
        for op in self.raw_ops:
            op.declare()
        env.store.materialize()
        self.chunk_ops = [fuse(c) if fuse is not None else list(c) for c in self.raw_chunks]
        self.chunk_segments = [split_segments(c) for c in self.chunk_ops]
        self.ops = [op for c in self.chunk_ops for op in c]
        self.segments = self.chunk_segments[0]

    def forward(self, st: Dict[str, torch.Tensor], chunk: int = 0) -> Dict[str, torch.Tensor]:
        for seg in self.chunk_segments[chunk]:
            seg.forward(st)
        return st

    def kernel_launch_estimate(self) -> int:
        return len(self.ops)
