"""Fusion of co-located neighbouring ops into single kernels.

A plan addresses ops individually, but ops that land in the same stage with the same (tp, dp, algo) and
the same recompute flag are executed by fused kernels:

  score, softmax, dropout, context            -> one flash-attention kernel        (AttentionCoreOp)
  GEMM(no bias), bias-dropout-residual        -> GEMM with epilogue                (FusedDenseDropAdd)
  MLP-GEMM-1, bias-act                        -> GEMM with bias + activation       (FusedUpAct)
  MLP-GEMM-1, bias-act, MLP-GEMM-2, dropout   -> MLPFn (activation derivative folded into a dgrad epilogue)

The fused objects reuse the member ops' parameters, so checkpoints and the per-op plan view do not
change.  With tensor parallelism the row-parallel GEMM's all-reduce sits between the GEMM and the
dropout-add, so those two stay separate kernels on the NCCL path.
"""
from __future__ import annotations

from typing import List, Sequence


from ..ops import functional as F
from ..parallel import mappings as M
from .base import Op
from .transformer_ops import (AttentionCoreOp, AttnDropoutOp, BiasActOp, BiasDropoutAddOp, ContextOp, DenseOp,
                              MLPUpOp, ScoreOp, SoftmaxOp)


class FusedGroup(Op):
    """Executes several member ops as one unit; reads/writes are the union seen from outside."""

    def __init__(self, members: Sequence[Op]):
        self.members = list(members)
        first = members[0]
        self.info, self.env, self.pl = first.info, first.env, first.pl
        self.tp_group, self.dp_group, self.local_bs = first.tp_group, first.dp_group, first.local_bs
        produced, reads = set(), []
        for m in members:
            for k in m.reads:
                if k not in produced and k not in reads:
                    reads.append(k)
            produced.update(m.writes)
        self.reads = tuple(reads)
        self.writes = tuple(sorted(produced))

    def declare(self):
        pass  # members declare their own parameters

    def required(self):
        out, produced = {}, set()
        for m in self.members:
            req = m.required()
            for k in m.reads:
                if k not in produced and k not in out and k in req:
                    out[k] = req[k]
            produced.update(m.writes)
        return out

    def produced(self):
        out = {}
        for m in self.members:
            out.update(m.produced())
        return out


class FusedAttention(FusedGroup):
    def __init__(self, members):
        super().__init__(members)
        score = members[0]
        self.core = AttentionCoreOp(score.info, score.env, mode=score.mode)
        self.core.sq, self.core.sk = score.sq, score.sk
        self.core._names = score._names        # the relative-position table, when the model has one
        self.reads = self.core.reads
        self.writes = ("x",)

    def forward(self, st):
        self.core.forward(st)


class FusedDenseDropAdd(FusedGroup):
    """residual + dropout(x W^T + b): one GEMM when tp == 1, GEMM -> all-reduce -> elementwise otherwise."""

    def forward(self, st):
        dense: DenseOp = self.members[0]
        c = self.env.cfg
        p_drop = c.hidden_dropout if self.env.training else 0.0
        w, b = dense.p(f"{dense.key}.weight"), dense.p(f"{dense.key}.bias")
        x, res = st["x"], st.pop("residual")
        if self.pl.tp == 1:
            st["x"] = F.linear(x, w, b, residual=res, dropout_p=p_drop, seed=self.seed())
        elif dense.info.algo == 0 and self.tpctx() is not None:
            st["x"] = F.row_parallel_linear_fused(x, w, b, res, p_drop, self.seed(), self.tpctx())
        elif dense.info.algo == 0:
            y = M.reduce_from_group(F.linear(x, w, None), self.tp_group)
            st["x"] = F.bias_dropout_add(y, b, res, p_drop, self.seed())
        else:
            y = F.linear(M.copy_to_group(x, self.tp_group), w, None)
            st["x"] = F.bias_dropout_add(y, b, res, p_drop, self.seed())


class FusedUpAct(FusedGroup):
    def accepts_dealt_out_rows(self) -> bool:
        return self.members[0].info.algo == 0

    def forward(self, st):
        up: MLPUpOp = self.members[0]
        w, b = up.p("dense_h_to_4h.weight"), up.p("dense_h_to_4h.bias")
        x = st["x"]
        if st.pop("_x_rows_dealt_out", False):
            st["x"] = F.gathered_column_linear_fused(x, w, b, self.env.cfg.activation, self.tpctx())
        elif up.info.algo == 0 and self.tpctx() is not None:
            st["x"] = F.column_parallel_linear_fused(x, w, b, self.env.cfg.activation, self.tpctx())
        elif up.info.algo == 0:
            st["x"] = F.linear(M.copy_to_group(x, self.tp_group), w, b, act=self.env.cfg.activation)
        else:
            y = M.reduce_from_group(F.linear(x, w, None), self.tp_group)
            st["x"] = F.bias_act(y, b, self.env.cfg.activation)


class FusedMLP(FusedGroup):
    """GEMM-1 + activation + GEMM-2 + dropout + residual (tp == 1: two forward kernels)."""

    def accepts_dealt_out_rows(self) -> bool:
        return self.members[0].info.algo == 0 and self.members[2].info.algo == 0

    def forward(self, st):
        up: MLPUpOp = self.members[0]
        down: DenseOp = self.members[2]
        c = self.env.cfg
        p_drop = c.hidden_dropout if self.env.training else 0.0
        w1, b1 = up.p("dense_h_to_4h.weight"), up.p("dense_h_to_4h.bias")
        w2, b2 = down.p(f"{down.key}.weight"), down.p(f"{down.key}.bias")
        x, res = st["x"], st.pop("residual")
        if st.pop("_x_rows_dealt_out", False):
            h = F.gathered_column_linear_fused(x, w1, b1, c.activation, self.tpctx())
            st["x"] = F.row_parallel_linear_fused(h, w2, b2, res, p_drop, self.seed(), self.tpctx())
        elif self.pl.tp == 1:
            st["x"] = F.mlp(x, w1, b1, w2, b2, residual=res, act=c.activation, dropout_p=p_drop, seed=self.seed())
        elif self.tpctx() is not None:
            h = F.column_parallel_linear_fused(x, w1, b1, c.activation, self.tpctx())
            st["x"] = F.row_parallel_linear_fused(h, w2, b2, res, p_drop, self.seed(), self.tpctx())
        else:
            h = F.linear(M.copy_to_group(x, self.tp_group), w1, b1, act=c.activation)
            y = M.reduce_from_group(F.linear(h, w2, None), self.tp_group)
            st["x"] = F.bias_dropout_add(y, b2, res, p_drop, self.seed())


def _same_place(ops: Sequence[Op]) -> bool:
    a = ops[0].info
    return all((o.info.tp, o.info.dp, o.info.recompute) == (a.tp, a.dp, a.recompute) for o in ops)


def fuse_ops(ops: List[Op]) -> List[Op]:
    """Greedy left-to-right pattern matching over the ops of one stage."""
    out: List[Op] = []
    i = 0
    n = len(ops)
    while i < n:
        o = ops[i]
        if isinstance(o, ScoreOp) and i + 3 < n and isinstance(ops[i + 1], SoftmaxOp) and \
                isinstance(ops[i + 2], AttnDropoutOp) and isinstance(ops[i + 3], ContextOp) and \
                _same_place(ops[i:i + 4]):
            out.append(FusedAttention(ops[i:i + 4]))
            i += 4
            continue
        if isinstance(o, MLPUpOp) and i + 3 < n and isinstance(ops[i + 1], BiasActOp) and \
                isinstance(ops[i + 2], DenseOp) and isinstance(ops[i + 3], BiasDropoutAddOp) and \
                _same_place(ops[i:i + 4]) and o.info.algo == 0 and ops[i + 2].info.algo == 0:
            out.append(FusedMLP(ops[i:i + 4]))
            i += 4
            continue
        # at tp > 1 the alternative partitioning (algo 1) leaves x in a layout the next op does not accept, so a
        # relayout has to run between the two ops and they cannot share a kernel
        if isinstance(o, MLPUpOp) and i + 1 < n and isinstance(ops[i + 1], BiasActOp) and _same_place(ops[i:i + 2]) \
                and (o.info.algo == 0 or o.info.tp == 1):
            out.append(FusedUpAct(ops[i:i + 2]))
            i += 2
            continue
        if isinstance(o, DenseOp) and i + 1 < n and isinstance(ops[i + 1], BiasDropoutAddOp) and \
                _same_place(ops[i:i + 2]) and (o.info.algo == 0 or o.info.tp == 1):
            out.append(FusedDenseDropAdd(ops[i:i + 2]))
            i += 2
            continue
        out.append(o)
        i += 1
    return out
