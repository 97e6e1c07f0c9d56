"""Uniform (Megatron-style) grid planner: the baseline the searched plans are compared with.

    python -m superscaler_b200.search.grid_plan --model-name gpt --model-size 1_3B ... --num-of-saved-configs 3

Enumerates pp x tp x dp x micro-batch x {full recompute, none} with layers split evenly over the stages,
scores each candidate with the same cost model and writes the best few as plan JSON
(reference: search/gen_megatron_plan.py:24-137).  The first and last op of a transformer are never
recomputed.  For T5 every split point between encoder stages and decoder stages is tried.
"""
from __future__ import annotations

import argparse
from typing import List

from .config import Plan, build_plan, save_plan
from .context import SearchContext, add_cli_arguments, args_from_namespace


def uniform_plans(ctx: SearchContext, pp: int, tp: int, dp: int, micro_bs: int, recompute: bool) -> List[Plan]:
    a = ctx.args
    ops = ctx.full_op_list
    n = len(ops)
    rc = [1 if recompute else 0] * n
    if a.model_name in ("gpt", "t5", "scale-layer", "bert", "vit"):
        rc[0] = rc[-1] = 0
    flat_tp, flat_dp, algo = [tp] * n, [dp] * n, [0] * n
    mk = lambda counts: build_plan(counts, flat_tp, flat_dp, rc, micro_bs, a.global_batch_size, ops, algo)  # noqa: E731
    L = a.num_layers
    if a.model_name in ("gpt", "scale-layer", "bert", "vit"):
        if L % pp:
            return []
        counts = [(L // pp) * 13] * pp
        counts[0] += 1
        counts[-1] += 2
        return [mk(counts)]
    if a.model_name == "t5":
        if pp == 1:
            return [mk([L * (13 + 21) + 5])]
        out = []
        for enc in range(1, pp):
            dec = pp - enc
            if L % enc == 0 and L % dec == 0:
                counts = [(L // enc) * 13] * enc
                counts[0] += 1
                counts[-1] += 1
                counts += [(L // dec) * 21] * dec
                counts[enc] += 1
                counts[-1] += 2
                out.append(mk(counts))
        return out
    if a.model_name == "resnet":
        counts = [(L // pp) * 8] * pp
        counts[0] += 4
        counts[-1] += 2
        counts[-1] += (L - (L // pp) * pp) * 8
        return [mk(counts)]
    raise ValueError(a.model_name)


def grid_search(ctx: SearchContext) -> List[Plan]:
    """All feasible uniform plans, fastest first (one per distinct predicted time, least memory wins ties)."""
    a = ctx.args
    by_time = {}
    for pp in range(a.start_num_stages, a.end_num_stages + 1):
        for tp in ctx.db.tp_list:
            if a.num_gpus % (pp * tp):
                continue
            dp = a.num_gpus // (pp * tp)
            for mbs in a.micro_batch_size:
                if mbs // dp not in a.micro_batch_size:
                    continue
                for recompute in (True, False):
                    for plan in uniform_plans(ctx, pp, tp, dp, mbs, recompute):
                        ctx.cost.evaluate(plan)
                        t, m = max(plan.time_list), max(plan.memory_list)
                        if m < a.memory_limit:
                            if t not in by_time or m < max(by_time[t].memory_list):
                                by_time[t] = plan
    return [by_time[t] for t in sorted(by_time)]


def best_uniform_plan(ctx: SearchContext, pp: int):
    """The fastest uniform plan with `pp` stages that fits the memory limit (None when there is none): the starting
    point `--initial-point grid` gives the search, so that what the search returns is never slower than the grid."""
    a = ctx.args
    best, best_t = None, float("inf")
    for tp in ctx.db.tp_list:
        if tp > a.max_tp or a.num_gpus % (pp * tp):
            continue
        dp = a.num_gpus // (pp * tp)
        for mbs in a.micro_batch_size:
            if mbs % dp or mbs // dp not in a.micro_batch_size or a.global_batch_size % mbs:
                continue
            for recompute in (False, True):
                for plan in uniform_plans(ctx, pp, tp, dp, mbs, recompute):
                    ctx.cost.evaluate(plan)
                    t = max(plan.time_list)
                    if max(plan.memory_list) < a.memory_limit and t < best_t:
                        best, best_t = plan, t
    return best


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_cli_arguments(p)
    args = args_from_namespace(p.parse_args(argv))
    ctx = SearchContext(args)
    plans = grid_search(ctx)
    if not plans:
        print("no feasible config")
        return
    for i, plan in enumerate(plans[:args.num_of_saved_configs]):
        t = max(plan.time_list)
        if args.config_save_path is None:       # nothing to write to: the prediction alone
            print(f"best_{i}: {t:.2f} ms, {max(plan.memory_list):.0f} MB (no --config-save-path: plan not saved)")
            continue
        path = f"{args.config_save_path}{args.model_name}_{args.model_size}_{args.num_layers}layers_megatron_est_{int(t)}.json"
        save_plan(plan, path, args.model_name, args.model_size, args.num_layers, getattr(args, "shapes", "reference"))
        print(f"best_{i}: {t:.2f} ms, {max(plan.memory_list):.0f} MB -> {path}")


if __name__ == "__main__":
    main()
