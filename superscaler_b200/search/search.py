"""Iterative bottleneck-alleviating plan search (CPU only).

    python -m superscaler_b200.search.search --model-name gpt --model-size 1_3B --global-batch-size 512 \
        --micro-batch-size 1 2 4 8 --num-nodes 1 --num-gpus-per-node 4 --memory-limit 12000 \
        --profiled-time-path <db>/ --config-save-path <out>/ --log-path <logs>/ --max-num-hops 7 \
        --time-budget-total 200

One search per pipeline-stage count (each in its own process), every search a sequence of trials; a
trial repeatedly picks the bottleneck stage and runs a multi-hop search over the primitives in policy
order until some plan beats the incumbent.  When a trial fails the search continues from the best
unexplored plan within 1.2x of the incumbent, then from already explored plans ("adaptive" phase).
Outputs per stage count: the plan JSON, a per-stage prediction CSV, trend CSVs; plus top_configs/ and a
summary CSV of the search cost (reference: search/aceso_search.py).
"""
from __future__ import annotations

import argparse
import csv
import os
import shutil
import time
from multiprocessing import Process, Queue
from typing import List, Optional

from .config import (BIG, Plan, balanced_plan, imbalanced_gpu_plan, imbalanced_op_plan, load_plan, save_plan,
                     write_stage_info_csv)
from .context import SearchArgs, SearchContext, add_cli_arguments, args_from_namespace, is_visited, mark_visited
from .policy import ordered_actions, pick_target_stage
from .primitives import action_table, finetune, finetune_stage_layouts


def initial_plan(ctx: SearchContext, num_stages: int) -> Optional[Plan]:
    a = ctx.args
    ops = ctx.full_op_list
    if a.initial_point == "balance":
        return balanced_plan(ops, num_stages, num_gpus=a.num_gpus, global_bs=a.global_batch_size,
                             micro_bs=a.micro_batch_size[0], max_tp=a.max_tp, flex_recompute=a.flex_recompute,
                             init_dim=a.init_dim)
    if a.initial_point == "imbalance_gpu":
        return imbalanced_gpu_plan(ops, num_stages, num_gpus=a.num_gpus, global_bs=a.global_batch_size,
                                   micro_batch_sizes=a.micro_batch_size, max_tp=a.max_tp)
    if a.initial_point == "imbalance_op":
        return imbalanced_op_plan(ops, num_stages, model_name=a.model_name, num_layers=a.num_layers,
                                  num_gpus=a.num_gpus, global_bs=a.global_batch_size, micro_bs=a.micro_batch_size[0],
                                  max_tp=a.max_tp, flex_recompute=a.flex_recompute)
    if a.initial_point == "grid":
        # not in the reference: start every stage count from its best uniform (Megatron-style) plan
        from .grid_plan import best_uniform_plan
        return best_uniform_plan(ctx, num_stages)
    return load_plan(a.initial_point, ops)[0]


def _best_of(plans: List[Plan], limit: float, extra=lambda p: True) -> Optional[Plan]:
    """Fastest plan that fits in memory; failing that, the one with the least memory."""
    best, best_t = None, BIG
    for p in plans:
        if max(p.time_list) < best_t and max(p.memory_list) <= limit and extra(p):
            best, best_t = p, max(p.time_list)
    if best is None:
        best_m = BIG
        for p in plans:
            if max(p.memory_list) < best_m and extra(p):
                best, best_m = p, max(p.memory_list)
    return best


def _sorted_plans(plans: List[Plan], metric: str) -> List[Plan]:
    """Stable insertion sort, ascending (ties keep arrival order)."""
    key = (lambda p: max(p.time_list)) if metric == "max_stage_time" else (lambda p: p.total_gpu_time)
    if metric not in ("max_stage_time", "total_gpu_time"):
        raise RuntimeError(f"sort_metric {metric} not supported.")
    out: List[Plan] = []
    for p in plans:
        for j in range(len(out)):
            if key(p) < key(out[j]):
                out.insert(j, p)
                break
        else:
            out.append(p)
    return out


class Searcher:
    def __init__(self, ctx: SearchContext):
        self.ctx = ctx
        self.table = action_table(ctx)

    def _note(self, plan: Plan, info: str) -> None:
        """Appends one line to the plan's history (kept because plan equality includes it)."""
        ops = [len(s.ops) for s in plan.stages]
        fmt = lambda ll: "[" + "".join(f"{max(x)}, " if min(x) == max(x) else f"{min(x)}~{max(x)}, " for x in ll) + "]"  # noqa: E731
        line = "{}|{:.2f}|{:.2f}| op = {}| tp = {} | dp = {} | algo = {} | rc = {} | gpus = {} | micro_bs = {} | time = {} | memory = {}".format(
            info, max(plan.time_list), max(plan.memory_list), ops, fmt([s.tp_size for s in plan.stages]),
            fmt([s.dp_size for s in plan.stages]), fmt([s.algo for s in plan.stages]),
            [sum(s.recompute_ops) for s in plan.stages], [s.num_gpus for s in plan.stages], plan.micro_bs,
            list(map(int, plan.time_list)), list(map(int, plan.memory_list)))
        self.ctx.debug(line)
        plan.history += line + "\n"

    def take_action(self, plan: Plan, target: int, prim) -> List[Plan]:
        ctx = self.ctx
        new = prim.apply_to(ctx, plan, target)
        out = []
        if new is not None and not is_visited(ctx.plan_visited, new.key()):
            ctx.cost.evaluate(new)
            out.append(new)
        return out

    def multi_hop(self, plan: Plan, hop: int, initial_time: float, adaptive: bool):
        ctx, a = self.ctx, self.ctx.args
        if ctx.trial_time_up() or ctx.total_time_up() or hop == a.max_num_hops:
            return None, None
        mark_visited(ctx.plan_visited, plan.key())
        if not adaptive:
            if a.adaptive_hyper_parameters > 0:
                ctx.explored_plans.append(plan)
            if a.continue_when_fail and plan in ctx.unexplored:
                ctx.unexplored.remove(plan)
        bottleneck = pick_target_stage(ctx, plan, adaptive=adaptive)
        if bottleneck is None:
            return None, None
        groups, _, _ = ordered_actions(ctx, plan, bottleneck, self.table)
        chain = [plan]
        for group in groups:
            produced: List[Plan] = []
            for prim in group:
                if ctx.trial_time_up() or ctx.total_time_up():
                    break
                for p in self.take_action(plan, bottleneck, prim):
                    produced.append(p)
                    self._note(p, f">>>> [CONFIG: target({bottleneck}), prim({prim.name})]\n")
            best_t, best = initial_time, None
            for p in produced:
                t, m = max(p.time_list), max(p.memory_list)
                if a.continue_when_fail and t < ctx.current_min_time * 1.2:
                    ctx.unexplored.append(p)
                if t < best_t and m <= a.memory_limit:
                    best_t, best = t, p
            if best is not None:
                return best, hop + 1
            for p in _sorted_plans(produced, a.sort_metric):
                chain.append(p)
                nxt, nxt_hop = self.multi_hop(p, hop + 1, initial_time, adaptive=False)
                if nxt is not None:
                    if max(nxt.time_list) < initial_time and max(nxt.memory_list) <= a.memory_limit:
                        return nxt, nxt_hop
                    chain.append(nxt)
        if a.continue_when_fail:
            return _best_of(chain, a.memory_limit), a.max_num_hops
        return None, None

    def trial(self, plan: Plan, adaptive: bool, initial_time: Optional[float] = None):
        ctx, a = self.ctx, self.ctx.args
        ctx.trial_clock.start()
        ctx.partner_visited = {}
        if initial_time is None:
            initial_time = BIG if max(plan.memory_list) > a.memory_limit else max(plan.time_list)
        max_targets = 1 if a.only_top_1_target else plan.num_stages
        tried = 0
        seen = [plan]
        while tried < max_targets:
            tried += 1
            new, hop = self.multi_hop(plan, 0, initial_time, adaptive)
            if new is not None:
                seen.append(new)
                if initial_time - max(new.time_list) > 0 and max(new.memory_list) <= a.memory_limit:
                    return new, tried, hop
        return _best_of(seen, a.memory_limit), max_targets, a.max_num_hops + 1

    def run(self, num_stages: int):
        ctx, a = self.ctx, self.ctx.args
        print(f"working on num_stages = {num_stages}")
        plan = initial_plan(ctx, num_stages)
        if plan is None:
            return None
        ctx.cost.refresh_recompute(plan)
        ctx.cost.evaluate(plan)
        self._note(plan, "start")
        ctx.current_min_time = max(plan.time_list) if max(plan.memory_list) < a.memory_limit else BIG
        ctx.explored = 0
        ctx.hit_resources = [0, 0, 0]
        ctx.unexplored, ctx.explored_plans = [], []
        ctx.total_clock.start()
        cur_mem = max(plan.memory_list)
        best = plan if max(plan.memory_list) < a.memory_limit else None
        n_trial = 0
        search_times = [0]
        trend = [ctx.current_min_time]
        targets_hist, hops_hist = [], []
        adaptive = False
        while n_trial < a.max_num_trials and sum(search_times) < a.time_budget_total:
            t0 = time.time()
            self._note(plan, f"\n[ Trial {n_trial} ] ")
            new, n_targets, n_hops = self.trial(plan, adaptive, ctx.current_min_time)
            search_times.append(time.time() - t0)
            for _ in range(a.finetune_after_trial):
                new = finetune(ctx, new)
                self._note(new, ">>>> [TMP CONFIG : (after finetune):\n")
            if a.finetune_tp_dp_after_trial:
                new = finetune_stage_layouts(ctx, new)
                self._note(new, ">>>> [TMP CONFIG : (after tune tp/dp) :\n")
            new_t, new_m = max(new.time_list), max(new.memory_list)
            trend.append(new_t)
            adaptive = False
            if (new_t < ctx.current_min_time and new_m <= a.memory_limit) or \
                    (cur_mem > a.memory_limit and new_m < cur_mem):
                cur_mem = new_m
                best = new.clone()
                plan = new
                if n_hops <= a.max_num_hops:
                    targets_hist.append(n_targets)
                    hops_hist.append(n_hops)
                if new_m <= a.memory_limit:
                    ctx.current_min_time = new_t
            else:
                if not a.continue_when_fail:
                    break
                plan = _best_of(ctx.unexplored, a.memory_limit)
                if plan is not None:
                    ctx.unexplored.remove(plan)
                else:
                    if a.adaptive_hyper_parameters <= 0:
                        break
                    adaptive = True
                    plan = _best_of(ctx.explored_plans, a.memory_limit,
                                    extra=lambda p: p.adaptive_times < a.adaptive_hyper_parameters)
                    if plan is None:
                        break
                    plan.adaptive_times += 1
            n_trial += 1
            if a.explored_budget is not None and ctx.explored >= a.explored_budget:
                break
        if best is not None and a.config_save_path is not None:
            path = f"{a.config_save_path}{a.model_name}_{a.model_size}_{best.num_stages}stages_{a.config_suffix}.json"
            save_plan(best, path, a.model_name, a.model_size, a.num_layers, getattr(a, "shapes", "reference"))
            print(f"config has been saved to {path}")
        self._report(best, num_stages, targets_hist, hops_hist, search_times, trend)
        mem = max(best.memory_list) if best is not None else 0
        return ctx.current_min_time, mem, ctx.explored, sum(search_times), list(ctx.hit_resources)

    def _report(self, best, num_stages, targets_hist, hops_hist, search_times, trend):
        ctx, a = self.ctx, self.ctx.args
        print(f"\n========== Best Result (num_stages = {num_stages}) ==========")
        if best is None:
            print("No feasible solution.")
        else:
            print(best.history)
            if a.config_save_path is not None:
                write_stage_info_csv(best, ctx.cost.reserved_list(best),
                                     f"{a.config_save_path}csv/info_{a.model_name}_{a.model_size}_{best.num_stages}stages_{a.config_suffix}.csv")
            if a.log_path is not None:
                with open(f"{a.log_path}trends/distribution_{a.model_name}_{a.model_size}_{best.num_stages}stages_{a.config_suffix}.csv",
                          "w", newline="") as f:
                    csv.writer(f).writerows([["num_targets"] + targets_hist, ["num_hops"] + hops_hist])
        accum, total = [], 0
        for i, t in enumerate(search_times):
            if i > 0:
                total += int(t + 1)
            accum.append(total)
        print(f"search time = {sum(search_times):.2f} s.  {accum} \nnum_explored_cases = {ctx.explored}")
        print(f"time trend: {list(map(int, trend))}\n")
        if a.log_path is not None:
            name = f"{a.log_path}trends/{a.model_name}_{a.model_size}_{num_stages}stages_init_{a.initial_point}_{a.max_num_hops}hops_{a.config_suffix}.csv"
            with open(name, "w", newline="") as f:
                csv.writer(f).writerows([["search_time (s)", "config time (ms)"]] + [[x, y] for x, y in zip(accum, trend)])


def search_stage_count(args: SearchArgs, num_stages: int):
    """One search for this stage count; with `--initial-point both` (not in the reference) two, from the balanced
    start and from the best uniform plan, of which the faster result and its saved plan are kept."""
    if args.initial_point != "both":
        return Searcher(SearchContext(args, verbose=False)).run(num_stages)
    import copy
    plan_file = None
    if args.config_save_path is not None:
        plan_file = f"{args.config_save_path}{args.model_name}_{args.model_size}_{num_stages}stages_{args.config_suffix}.json"
    best, kept = None, None
    for start in ("balance", "grid"):
        one = copy.copy(args)
        one.initial_point = start
        res = Searcher(SearchContext(one, verbose=False)).run(num_stages)
        better = res is not None and 0 < res[0] < BIG and (best is None or res[0] < best[0])
        if better:
            best = res
            if plan_file is not None and os.path.exists(plan_file):
                kept = plan_file + ".best"
                shutil.copy(plan_file, kept)
        elif best is None and res is not None:
            best = res
    if kept is not None:
        shutil.move(kept, plan_file)
    return best


def _worker(args: SearchArgs, num_stages: int, queue) -> None:
    res = search_stage_count(args, num_stages)
    d = queue.get()
    d[num_stages] = res
    queue.put(d)


def run_all(args: SearchArgs) -> dict:
    """Searches every stage count in [start, end]; returns {num_stages: (time, mem, explored, cost, hits)}."""
    for sub in ("top_configs", "csv"):
        if args.config_save_path is not None:
            os.makedirs(os.path.join(args.config_save_path, sub), exist_ok=True)
    if args.log_path is not None:
        os.makedirs(os.path.join(args.log_path, "trends"), exist_ok=True)
    results: dict = {}
    counts = range(args.start_num_stages, args.end_num_stages + 1)
    if args.multi_process:
        q: Queue = Queue()
        q.put(results)
        procs = [Process(target=_worker, args=(args, n, q)) for n in counts]
        for p in procs:
            p.start()
        for p in procs:
            p.join()
        results = q.get()
    else:
        for n in counts:
            results[n] = search_stage_count(args, n)
    return results


def save_top_plans(results: dict, args: SearchArgs) -> List[list]:
    ranked = sorted((r[0], n) for n, r in results.items() if r is not None and r[0] > 0 and r[0] < BIG)
    rows = []
    span = args.end_num_stages - args.start_num_stages + 1
    for t, n in ranked[:min(span, args.num_of_saved_configs)]:
        src = f"{args.config_save_path}{args.model_name}_{args.model_size}_{n}stages_{args.config_suffix}.json"
        dst = f"{args.config_save_path}top_configs/{args.model_name}_{args.model_size}_{n}stages_{args.config_suffix}.json"
        if os.path.exists(src):
            shutil.copy(src, dst)
        _, mem, explored, _, _ = results[n]
        rows.append([n, f"{t / 1000:.2f}", f"{args.global_batch_size / (t / 1000):.2f}", f"{mem:.0f}", f"{explored}"])
    header = ["# of stages", "est_iteration_time(s)", "est_thpt(samples/s)", "est_mem(MB)", "# of explored cases"]
    print("\t".join(header))
    for r in rows:
        print("\t".join(str(x) for x in r))
    return rows


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_cli_arguments(p)
    args = args_from_namespace(p.parse_args(argv))
    t0 = time.time()
    results = run_all(args)
    cost = time.time() - t0
    if args.config_save_path is not None:
        save_top_plans(results, args)
    if args.log_path is not None:
        with open(f"{args.log_path}{args.model_name}_{args.model_size}_summary_{args.config_suffix}.csv", "w", newline="") as f:
            csv.writer(f).writerows([["search_cost"], [f"{cost:.2f}"]])
    print(f"\noverall search time: {cost:.2f} s")


if __name__ == "__main__":
    main()
