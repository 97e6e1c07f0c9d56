"""Stage optimizer over the flat parameter buffers: data-parallel gradient reduction, global gradient
norm, clipping, Adam / SGD update and bf16 copy-out in fused kernels, with no host synchronisation.

Replaces the reference chain LocalDDP.allreduce_gradients -> copy model grads to main grads ->
unscale / inf check -> clip_grad_norm_fp32 -> apex FusedAdam -> copy main params to model params
(runtime/megatron/model/distributed.py:195-263, runtime/megatron/optimizer/optimizer.py:348-443,
runtime/megatron/optimizer/clip_grads.py:29-120).

Gradient norm: every unique parameter element must be counted once.  A parameter replicated over a TP
group of size t and a DP group of size d exists t * d times in the job, a TP-sharded one d times, so each
rank weights its local sum of squares by 1 / copies before the all-reduce over the whole job.  (The
reference all-reduces unweighted sums over the world group, clip_grads.py:79-81,106-108.)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import native
from .params import ParamStore


def _merge(ranges: List[Tuple[int, int]]) -> List[Tuple[int, int]]:
    out: List[Tuple[int, int]] = []
    for off, n in sorted(ranges):
        if out and out[-1][0] + out[-1][1] == off:
            out[-1] = (out[-1][0], out[-1][1] + n)
        else:
            out.append((off, n))
    return out


class StageOptimizer:
    def __init__(self, store: ParamStore, pstate, *, lr=1.5e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 clip_grad=1.0, kind="adam", momentum=0.9, norm_exclude=()):
        self.store, self.pstate = store, pstate
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.clip_grad, self.kind, self.momentum = clip_grad, kind, momentum
        self.step_count = 0
        dev = store.device
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.skipped = torch.zeros(1, dtype=torch.int32, device=dev)
        self.grad_norm_sq = self.sumsq
        # ranges grouped by the number of copies of the parameter in the job
        groups: Dict[int, List[Tuple[int, int]]] = {}
        for s in store.specs:
            if s.name in norm_exclude:
                continue  # a non-root copy of a tied weight: its (identical) gradient is counted at the root
            off, n = store.offsets[s.name]
            replicated_over_tp = s.tp > 1 and s.shard_dim is None
            copies = s.dp * (s.tp if replicated_over_tp else 1)
            groups.setdefault(copies, []).append((off, (n + 127) // 128 * 128))
        self._norm_exclude = set(norm_exclude)
        self.norm_groups = {c: _merge(r) for c, r in groups.items()}
        self.dp_buckets = store.buckets_by_dp()
        # Sharded update (pure data-parallel stage with peer-mapped gradient AND model buffers): the weight-decay
        # part [0, wd_end) of the flat buffers, which holds all the large matrices, is reduce-SCATTERED; every rank
        # runs Adam on its slice only and writes the new bf16 weights into every rank's model buffer.  Half the
        # NVLink bytes of an all-reduce and 1 / dp of the optimizer work.  The small tail [wd_end, total) (biases,
        # LayerNorm / BatchNorm parameters, some of which the model reads from the fp32 master buffer) stays
        # replicated: all-reduced and updated on every rank.  Master weights and moments outside a rank's slice
        # go stale; `sync_replicas()` refreshes them before a checkpoint is written.
        self.sharded = store.symm_grad is not None and store.symm_model16 is not None and store.wd_end >= 8 * 128
        if self.sharded:
            self.shard_lo, self.shard_hi = store.symm_grad.slice_of(store.wd_end)
            self._partials = torch.zeros(native.ext().comm_max_blocks(), dtype=torch.float32, device=dev)
            self._tail_sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
            self._skipped_tail = torch.zeros(1, dtype=torch.int32, device=dev)   # the slice's launch does the counting
        self._replicas_stale = False

    # ---- data-parallel gradient reduction (NCCL path) -----------------------------------------
    def reduce_gradients(self) -> None:
        """Average gradients over each op's DP group.  With a peer-mapped gradient buffer (pure data-parallel
        stage) ONE fused kernel sums over the ranks and applies 1/dp through NVSwitch; otherwise one NCCL
        all-reduce per contiguous (tp, dp) range."""
        if self.sharded:
            sg, st = self.store.symm_grad, self.store
            sg.reduce_scatter_scale_sumsq_(st.wd_end, 1.0 / sg.world, self._partials)
            if st.total > st.wd_end:
                sg.allreduce_scale_(st.total - st.wd_end, 1.0 / sg.world, offset=st.wd_end)
            return
        if self.store.symm_grad is not None:
            self.store.symm_grad.allreduce_scale_(self.store.total, 1.0 / self.store.symm_grad.world)
            return
        for (tp, dp), ranges in self.dp_buckets.items():
            if dp == 1:
                continue
            pl = self.pstate.placement(tp, dp)
            group = self.pstate.group(pl.dp_ranks)
            for off, n in ranges:
                buf = self.store.grad[off:off + n]
                buf.mul_(1.0 / dp)
                dist.all_reduce(buf, group=group)

    # ---- norm + update ----------------------------------------------------------------------
    def _global_sumsq(self) -> torch.Tensor:
        g = self.store.grad
        if self.sharded:
            # this rank's slice counts once (the slices partition the buffer), the replicated tail 1 / dp times
            st = self.store
            world = st.symm_grad.world
            if st.total > st.wd_end:
                native.ext().sumsq(g[st.wd_end:st.total], self._tail_sumsq, False)
                torch.add(self._partials.sum(), self._tail_sumsq[0], alpha=1.0 / world, out=self.sumsq[0])
            else:
                self.sumsq[0] = self._partials.sum()
            dist.all_reduce(self.sumsq)
            return self.sumsq
        first = True
        if g.is_cuda:
            ext = native.ext()
            for copies, ranges in self.norm_groups.items():
                for off, n in ranges:
                    if copies == 1:
                        ext.sumsq(g[off:off + n], self.sumsq, not first)
                    else:
                        tmp = torch.zeros(1, dtype=torch.float32, device=g.device)
                        ext.sumsq(g[off:off + n], tmp, False)
                        if first:
                            self.sumsq.copy_(tmp / copies)
                        else:
                            self.sumsq.add_(tmp / copies)
                    first = False
        else:
            total = torch.zeros(1, dtype=torch.float32)
            for copies, ranges in self.norm_groups.items():
                for off, n in ranges:
                    total += (g[off:off + n] ** 2).sum() / copies
            self.sumsq.copy_(total)
        if self.pstate.world_size > 1:
            dist.all_reduce(self.sumsq)
        return self.sumsq

    def step(self, lr: Optional[float] = None, grad_scale: float = 1.0, zero_grad: bool = True) -> None:
        lr = self.lr if lr is None else lr
        self.step_count += 1
        st = self.store
        sumsq = self._global_sumsq()
        if self.sharded:
            ext = native.ext()
            lo, hi = self.shard_lo, self.shard_hi
            for a, b, wd_end, skipped in ((lo, hi, hi - lo, self.skipped), (st.wd_end, st.total, 0, self._skipped_tail)):
                if b <= a:
                    continue
                if self.kind == "adam":
                    ext.adam_step(st.master[a:b], st.exp_avg[a:b], st.exp_avg_sq[a:b], st.grad[a:b], st.model16[a:b],
                                  sumsq, skipped, lr, self.betas[0], self.betas[1], self.eps, self.wd,
                                  self.step_count, grad_scale, self.clip_grad, wd_end, zero_grad)
                else:
                    ext.sgd_step(st.master[a:b], st.exp_avg[a:b], st.grad[a:b], st.model16[a:b], sumsq, skipped,
                                 lr, self.momentum, self.wd, grad_scale, self.clip_grad, wd_end, zero_grad,
                                 self.step_count == 1)
            st.symm_model16.allgather_(st.wd_end)
            self._replicas_stale = True
            return
        if st.grad.is_cuda:
            ext = native.ext()
            if self.kind == "adam":
                ext.adam_step(st.master, st.exp_avg, st.exp_avg_sq, st.grad, st.model16, sumsq, self.skipped, lr,
                              self.betas[0], self.betas[1], self.eps, self.wd, self.step_count, grad_scale,
                              self.clip_grad, st.wd_end, zero_grad)
            else:
                ext.sgd_step(st.master, st.exp_avg, st.grad, st.model16, sumsq, self.skipped, lr, self.momentum,
                             self.wd, grad_scale, self.clip_grad, st.wd_end, zero_grad, self.step_count == 1)
            return
        # CPU restatement
        norm = float(sumsq.sqrt()) * grad_scale
        if not math.isfinite(norm):       # as the kernels do: a step with inf / nan gradients changes nothing
            self.skipped += 1
            if zero_grad:
                st.grad.zero_()
            return
        clip = min(1.0, self.clip_grad / (norm + 1e-6)) if self.clip_grad > 0 else 1.0
        g = st.grad * (grad_scale * clip)
        wd = torch.zeros_like(g)
        wd[:st.wd_end] = self.wd
        if self.kind == "adam":
            b1, b2 = self.betas
            st.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
            st.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
            bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
            denom = st.exp_avg_sq.sqrt() / (bc2 ** 0.5) + self.eps
            st.master.sub_(lr * ((st.exp_avg / bc1) / denom + wd * st.master))
        else:
            g = g + wd * st.master
            if self.step_count == 1:
                st.exp_avg.copy_(g)
            else:
                st.exp_avg.mul_(self.momentum).add_(g)
            st.master.sub_(lr * st.exp_avg)
        st.model16.copy_(st.master.to(torch.bfloat16))
        if zero_grad:
            st.grad.zero_()

    def grad_norm(self) -> float:
        """Host read of the last global gradient norm (synchronises)."""
        return float(self.sumsq.sqrt())

    def skipped_steps(self) -> int:
        """Steps left out so far because the gradients held inf or nan (host read, synchronises)."""
        return int(self.skipped)

    def _per_parameter_total(self, value_of) -> float:
        """Sum over the whole model of `value_of(spec, offset, numel)`, every parameter counted once however many
        ranks hold a copy of it (the weights the norm groups use), reduced over the job."""
        total = torch.zeros(1, dtype=torch.float64)
        for s in self.store.specs:
            if s.name in self._norm_exclude:
                continue
            off, n = self.store.offsets[s.name]
            copies = s.dp * (s.tp if (s.tp > 1 and s.shard_dim is None) else 1)
            total += float(value_of(s, off, n)) / copies
        if self.pstate.world_size > 1:
            t = total.to(self.store.device)
            dist.all_reduce(t)
            total = t.cpu()
        return float(total)

    def count_zeros_in_grad(self) -> int:
        """Zero entries of the (reduced) gradients of the whole model; call it between `reduce_gradients` and
        `step` (reference: count_zeros_fp32, runtime/megatron/optimizer/clip_grads.py:123-148).  With the sharded
        update only this rank's slice of the large matrices is reduced, so the count is taken before sharding is
        of use: it is refused there."""
        assert not self.sharded, "--log-num-zeros-in-grad needs the unsharded update (Trainer(shard_optimizer=False))"
        g = self.store.grad
        return int(round(self._per_parameter_total(lambda s, off, n: (g[off:off + n] == 0).sum())))

    def params_norm(self) -> float:
        """L2 norm of the model's parameters, as the model computes with them (bf16 weights, fp32 norm
        parameters); reference: calc_params_l2_norm, runtime/megatron/utils.py:59-84."""
        params = self.store.params
        return math.sqrt(self._per_parameter_total(lambda s, off, n: params[s.name].detach().float().pow(2).sum()))

    def sync_replicas(self) -> None:
        """After sharded steps: every rank fetches the other ranks' slices of the fp32 master weights and of the
        moments (NCCL broadcasts, collective), so that any rank can write a complete checkpoint."""
        if not self.sharded or not self._replicas_stale:
            return
        sg, st = self.store.symm_grad, self.store
        for r in range(sg.world):
            lo, hi = (int(x) for x in native.ext().comm_slice(st.wd_end, sg.world, r))
            if hi <= lo:
                continue
            bufs = [st.master, st.exp_avg] + ([st.exp_avg_sq] if self.kind == "adam" else [])
            for buf in bufs:
                dist.broadcast(buf[lo:hi], src=dist.get_global_rank(sg.group, r), group=sg.group)
        self._replicas_stale = False

    def state_dict(self) -> dict:
        self.sync_replicas()
        return {"step": self.step_count, "exp_avg": self.store.exp_avg.clone(), "exp_avg_sq": self.store.exp_avg_sq.clone(),
                "master": self.store.master.clone()}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd["step"]
        self.store.exp_avg.copy_(sd["exp_avg"])
        self.store.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.store.master.copy_(sd["master"])
        self.store.model16.copy_(self.store.master.to(torch.bfloat16))
