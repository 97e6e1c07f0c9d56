"""Model = flat list of named ops; a pipeline stage owns a contiguous slice of it.

Same representation as the reference (runtime/megatron/model/flex_gpt.py:59-78,
runtime/megatron/model/module.py:180-251): every op carries its own tensor-parallel degree, data-parallel
degree, partition algorithm and recompute flag.  Ops communicate through a small dict of named tensors
(`state`): "x" is the main activation, other keys ("residual", "bias", "value", "enc_out", ...) are the
reference's "extra tensors" that skip over ops.  Each op lists the keys it reads and writes, which
gives the set of tensors that crosses a stage boundary by a liveness pass instead of hand-written
send/recv offsets (runtime/megatron/model/flex_model.py:180-209).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Sequence, Tuple

import torch

from ..ops import functional as F
from ..parallel.state import OpPlacement, ParallelState
from ..runtime.params import ParamSpec, ParamStore


@dataclass
class OpInfo:
    name: str
    index: int          # position in the full op list
    layer: int          # layer number (or -1), used for seeding and scale factors
    tp: int = 1
    dp: int = 1
    algo: int = 0
    recompute: int = 0


@dataclass
class Env:
    """Everything an op needs at build time besides its OpInfo."""
    cfg: Any                         # model hyper-parameters (see models/gpt.py etc.)
    pstate: ParallelState
    store: ParamStore
    micro_bs: int                    # stage-aggregate micro batch size of the plan
    fused_comm: bool = False         # use the in-kernel peer-memory collectives where available
    distribute_saved_activations: bool = False   # recompute segments keep 1 / tp of inputs replicated over tp
    stage_ops: Sequence[OpInfo] = ()
    tp_contexts: Dict[Tuple[int, ...], Any] = field(default_factory=dict)

    def tp_context(self, pl: OpPlacement, local_bs: int):
        """Symmetric scratch for the fused GEMM + all-reduce kernel of this op's tensor-parallel group, or None
        when the NCCL path is to be used (tp == 1, CPU tensors, a group that spans nodes and so cannot map peer
        memory, or fused communication switched off).  Created
        on first use; all ranks of the group reach that point together because they execute the same plan."""
        if not self.fused_comm or pl.tp == 1 or self.store.device.type != "cuda":
            return None
        if not self.pstate.same_node(pl.tp_ranks):
            return None
        key = tuple(pl.tp_ranks)
        ctx = self.tp_contexts.get(key)
        if ctx is None:
            from ..parallel.symm import FusedTPContext
            c = self.cfg
            seq = max(getattr(c, "seq_length", 1), getattr(c, "dec_seq_length", 1))
            ctx = FusedTPContext(self.group(pl.tp_ranks), local_bs * seq, c.hidden, self.store.device)
            self.tp_contexts[key] = ctx
        return ctx

    def placement(self, info: OpInfo) -> OpPlacement:
        return self.pstate.placement(info.tp, info.dp)

    def group(self, ranks):
        return self.pstate.group(ranks)


class Op:
    """Base class.  Subclasses set `reads` / `writes` and implement declare() and forward()."""
    reads: Tuple[str, ...] = ("x",)
    writes: Tuple[str, ...] = ("x",)

    def __init__(self, info: OpInfo, env: Env):
        self.info, self.env = info, env
        self.pl = env.placement(info)
        self.tp_group = env.group(self.pl.tp_ranks)
        self.dp_group = env.group(self.pl.dp_ranks)
        self.local_bs = env.micro_bs // info.dp
        self._names: Dict[str, str] = {}

    # -- parameters ---------------------------------------------------------------------------
    def declare(self) -> None:
        """Registers the op's ParamSpecs with self.env.store (via self.param_spec)."""

    def param_spec(self, key: str, shape, init, *, full_shape=None, shard_dim=None, std=0.02, weight_decay=True,
                   fp32=False, seed_key=None, shared_key=None) -> None:
        name = f"ops.{self.info.index}.{key}"
        spec = ParamSpec(name=name, shape=tuple(shape), init=init, std=std, weight_decay=weight_decay, fp32=fp32,
                         full_shape=tuple(full_shape) if full_shape is not None else None, shard_dim=shard_dim,
                         tp=self.pl.tp, tp_rank=self.pl.tp_rank, dp=self.pl.dp,
                         seed_key=seed_key or f"{self.info.name}.{self.info.layer}.{key}", shared_key=shared_key)
        self._names[key] = self.env.store.declare(spec)

    def p(self, key: str) -> torch.nn.Parameter:
        return self.env.store[self._names[key]]

    # -- layouts (see models/static_info.py) ---------------------------------------------------
    def required(self) -> Dict[str, Any]:
        from .static_info import required_layouts
        return required_layouts(self.info.name, self.info.algo)

    def produced(self) -> Dict[str, Any]:
        from .static_info import produced_layouts
        return produced_layouts(self.info.name, self.info.algo)

    # -- execution ----------------------------------------------------------------------------
    def forward(self, st: Dict[str, torch.Tensor]) -> None:
        raise NotImplementedError

    def tpctx(self):
        return self.env.tp_context(self.pl, self.local_bs)

    def seed(self, sharded: bool = False) -> int:
        """Dropout seed: equal across a TP group for replicated tensors, distinct across DP ranks."""
        s = F.seed_state().next()
        s = (s + 0x632BE59BD9B4E019 * (self.pl.dp_rank + 1)) & ((1 << 62) - 1)
        if sharded:
            s = (s + 0x9E6C63D0676A9A99 * (self.pl.tp_rank + 1)) & ((1 << 62) - 1)
        return s


def boundary_keys(ops: Sequence[Op], cut: int, always: Sequence[str] = ()) -> List[str]:
    """Keys that are live across the boundary before op `cut`: read by some op >= cut before being rewritten,
    and written by some op < cut (or supplied by the data loader on both sides and therefore not sent)."""
    written_before = set()
    for op in ops[:cut]:
        written_before.update(op.writes)
    live, killed = [], set()
    for op in ops[cut:]:
        for k in op.reads:
            if k not in killed and k in written_before and k not in live:
                live.append(k)
        killed.update(op.writes)
    for k in always:
        if k not in live:
            live.append(k)
    return live
