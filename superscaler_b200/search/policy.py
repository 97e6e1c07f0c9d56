"""Bottleneck selection and action ordering of the iterative search.

  target stage  : the stage with the largest memory when the plan is out of memory, else the largest time;
                  each (plan, stage) pair is tried once
  partner stage : the stage with the most "efficient idle time" (or the least memory) to absorb moved work
  action order  : primitive groups ordered by which of {ideal compute, efficiency loss, recompute} dominates
                  the bottleneck, filtered by the sign each primitive has on time / memory / comm
(reference: search/aceso_policy.py:23-208).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

from .config import BIG, Plan
from .context import SearchContext, is_visited, mark_visited, num_visited

ALL = ("+", "-", "0")


def pick_target_stage(ctx: SearchContext, plan: Plan, metric=None, tag: str = "", adaptive=False) -> Optional[int]:
    key = (plan.key(), tag)
    if not adaptive and num_visited(ctx.target_visited, key) >= plan.num_stages:
        return None
    values = plan.memory_list if (metric is None and max(plan.memory_list) > ctx.args.memory_limit) else plan.time_list
    best, best_v = None, 0
    for i in range(plan.num_stages):
        if values[i] > best_v and (adaptive or not is_visited(ctx.target_visited, key, i)):
            best, best_v = i, values[i]
    if best is not None:
        mark_visited(ctx.target_visited, key, best)
    return best


def pick_partner_stage(ctx: SearchContext, plan: Plan, action: str, partner_action: str, target: Optional[int],
                       metric: str = "time_with_efficiency", tag: str = "") -> Optional[int]:
    key = (plan.key(), action, partner_action, str(target), str(tag))
    if num_visited(ctx.partner_visited, key) >= plan.num_stages - 1:
        return None
    partner = None
    if metric == "time_with_efficiency":
        best = 0
        for i, v in enumerate(plan.efficient_time_list):
            if v > best and not is_visited(ctx.partner_visited, key, i) and i != target:
                partner, best = i, v
    elif metric == "memory":
        best = BIG
        for i, v in enumerate(plan.memory_list):
            if v < best and not is_visited(ctx.partner_visited, key, i) and i != target:
                partner, best = i, v
    else:
        raise RuntimeError(f"metric {metric} for partner selection is not supported.")
    if partner is not None:
        mark_visited(ctx.partner_visited, key, partner)
    return partner


def filter_actions(table, memory=ALL, efficiency=ALL, time=ALL, comm=ALL, gpus=ALL, workloads=ALL, exclude=()):
    return [p for p in table if p not in exclude and p.memory in memory and p.time in time and
            p.efficiency in efficiency and p.comm in comm and p.num_devices in gpus and p.workloads in workloads]


def _share(values: Sequence[float], i: int) -> float:
    return values[i] / sum(values) if values[i] > 0 else 0


def ordered_actions(ctx: SearchContext, plan: Plan, bottleneck: int, table) -> tuple:
    """Returns (list of action groups in the order to try, turn-back actions (unused), stage type)."""
    if ctx.args.random_order_actions:
        names = ["move_out", "inc_dp", "dec_dp", "inc_tp", "dec_tp", "inc_mbs", "dec_mbs"]
        return [[names[i]] for i in ctx.rng.sample(range(7), 7)], [], ""
    if max(plan.memory_list) > ctx.args.memory_limit:
        return [filter_actions(table, memory=("-",))], [], "OOM"
    n = plan.num_stages
    comp, loss, rc = plan.ideal_time_per_gpu, plan.eff_loss_time_per_gpu, plan.recomp_time_per_gpu
    comp_t, loss_t, rc_t = comp[bottleneck], loss[bottleneck], rc[bottleneck]
    avg_comp, avg_loss = sum(comp) / n, sum(loss) / n
    comp_r, loss_r, rc_r = _share(comp, bottleneck), _share(loss, bottleneck), _share(rc, bottleneck)
    ratios = [comp_r, loss_r, rc_r]
    groups: List[list] = []
    seen: list = []

    def take(**kw):
        got = filter_actions(table, exclude=seen, **kw)
        groups.append(got)
        seen.extend(got)

    less_comm = ("-", "0") if loss_t > avg_loss else ALL
    less_time = ("-", "0") if comp_t > avg_comp else ALL
    less_mem = ("-", "0") if rc_t > 0 else ALL
    for rank in range(3):
        top = max(ratios)
        if comp_r == top:      # compute bound: shrink time
            take(time=("-",), comm=less_comm, memory=less_mem)
            take(time=("-",))
            ratios.remove(comp_r)
            if rank == 0:
                ctx.hit_resources[0] += 1
        elif loss_r == top:    # efficiency-loss bound: shrink communication
            take(time=less_time, comm=("-",), memory=less_mem)
            take(comm=("-",))
            ratios.remove(loss_r)
            if rank == 0:
                ctx.hit_resources[1] += 1
        elif rc_r == top:      # recompute bound: shrink memory
            take(time=less_time, comm=less_comm, memory=("-",))
            take(memory=("-",))
            ratios.remove(rc_r)
            if rank == 0:
                ctx.hit_resources[2] += 1
    groups.append(filter_actions(table, exclude=seen))
    return groups, [], ""
