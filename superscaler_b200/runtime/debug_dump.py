"""Per-rank debug files: what every op produced and what every parameter's gradient looks like.

The reference writes such files when DEBUG_OUTPUT / DEBUG_GRAD are set in the environment (print_tensors from the
post-forward hook, runtime/megatron/model/flex_model.py:245-247; weights and gradients before and after the
shared-weight sync, runtime/megatron/training.py:700-722) and compares them by eye across plans.  Here the entry
point's `--debug-dump output|grad|all` (with --log-path) writes one line per tensor with its shape and three
statistics instead of the values, so two plans of one model can be compared with `diff`:

    <log-path><plan>_debug_output_rank_<r>.log    iteration, op index, op name, key, shape, mean, largest magnitude, norm
    <log-path><plan>_debug_grad_rank_<r>.log      iteration, parameter, shape, weight norm, gradient norm

Reading the statistics synchronises with the device after every op: a debugging aid, not for timed runs.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import stage


def _stats(t: torch.Tensor) -> str:
    f = t.detach().float()
    if f.numel() == 0:
        return "empty"
    return f"mean {float(f.mean()):+.6e} | max {float(f.abs().max()):.6e} | norm {float(f.norm()):.6e}"


class DebugDump:
    def __init__(self, trainer, log_path: str, plan_name: str, what: str = "all", iterations: int = 1):
        assert what in ("output", "grad", "all")
        os.makedirs(log_path, exist_ok=True)
        self.trainer, self.what, self.iterations = trainer, what, iterations
        stem = os.path.join(log_path, f"{plan_name}_debug_")
        self.out_path = f"{stem}output_rank_{trainer.rank}.log"
        self.grad_path = f"{stem}grad_rank_{trainer.rank}.log"
        for path in (self.out_path, self.grad_path):
            open(path, "w").close()
        self._out: Optional[object] = None
        if what in ("output", "all"):
            self._out = open(self.out_path, "a")
            stage.AFTER_OP_HOOKS.append(self._after_op)

    def active(self) -> bool:
        return self.trainer.iteration < self.iterations

    def _after_op(self, op, st) -> None:
        if not self.active() or self._out is None:
            return
        for key in op.writes:
            t = st.get(key)
            if isinstance(t, torch.Tensor):
                self._out.write(f"it {self.trainer.iteration} | op {op.info.index:4d} {op.info.name} | {key} "
                                f"{tuple(t.shape)} | {_stats(t)}\n")

    def gradients(self, when: str) -> None:
        """Call between the gradient reduction and the optimizer step (`when` names the point)."""
        if not self.active() or self.what not in ("grad", "all"):
            return
        store = self.trainer.store
        with open(self.grad_path, "a") as f:
            f.write(f"=== iteration {self.trainer.iteration}, {when} ===\n")
            for name, p in store.params.items():
                g = p.main_grad
                f.write(f"it {self.trainer.iteration} | {name} {tuple(p.shape)} | weight norm "
                        f"{float(p.detach().float().norm()):.6e} | grad norm {float(g.norm()):.6e}\n")

    def close(self) -> None:
        if self._out is not None:
            if self._after_op in stage.AFTER_OP_HOOKS:
                stage.AFTER_OP_HOOKS.remove(self._after_op)
            self._out.close()
            self._out = None
