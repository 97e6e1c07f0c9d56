"""Search primitives (actions on a plan) and the fine-tuning passes.

  dec_op            : migrate ops from the bottleneck towards a partner stage, stage by stage, until the
                      bottleneck's predicted time (or memory) meets a goal between the two stages' values
  inc/dec_tp, _dp   : move GPUs between stages (one stage halves a degree, others double one) while the
                      plan stays legal
  inc/dec_mbs       : next / previous micro-batch size, re-picking the best tp x dp of every stage
  inc_tp_dec_dp ... : optional exchange of degrees inside one stage
Each primitive carries the sign of its effect on time, memory, #devices, workload, efficiency and
communication, which the policy filters on (reference: search/aceso_prims.py:812-826).
"""
from __future__ import annotations

from typing import List, Optional

from .config import BIG, Plan, StagePlan, is_legal
from .context import SearchContext
from .policy import pick_partner_stage, pick_target_stage


class Primitive:
    def __init__(self, name, time, memory, num_devices, workloads, efficiency, comm, func):
        self.name, self.time, self.memory, self.num_devices = name, time, memory, num_devices
        self.workloads, self.efficiency, self.comm, self.func = workloads, efficiency, comm, func

    def apply_to(self, ctx: SearchContext, plan: Plan, bottleneck: int) -> Optional[Plan]:
        return self.func(ctx, plan, bottleneck, self.name)


# ------------------------------------------------------------------------------------------------
# op migration
# ------------------------------------------------------------------------------------------------
def _migration_goals(ctx, plan, bottleneck, partner, metric):
    if metric in ("time", "time_with_efficiency"):
        t = plan.compute_time_list
        ratios = [1, 0.8, 0.6, 0.4, 0.2, 0] if ctx.args.simple_prim_mig else [0.4, 0.2, 0]
        gap = t[bottleneck] - t[partner]
        return [t[bottleneck] - gap * r for r in ratios]
    if metric == "memory":
        return [ctx.args.memory_limit]
    raise RuntimeError(f"metric {metric} not implemented.")


def move_ops_once(ctx: SearchContext, plan: Plan, src: int, towards: int, count: int = 1, src_recompute=None) -> Plan:
    """Moves `count` ops from stage `src` to its neighbour in the direction of `towards` (memoised)."""
    memo_key = (plan.key(), src, towards, count)
    hit = ctx.move_memo.get(memo_key)
    if hit is not None:
        out = hit.clone()
        out.history = plan.history
        return out
    if count == 0:
        return plan
    if len(plan.stages[src].ops) <= count:
        return plan
    new = plan.clone()
    s = new.stages[src]
    if src < towards:
        d = new.stages[src + 1]
        d.ops = s.ops[-count:] + d.ops
        d.recompute_ops = [0] * count + d.recompute_ops
        s.ops = s.ops[:-count]
        s.recompute_ops = s.recompute_ops[:-count]
        d_tp, d_dp = d.tp_size[0], d.dp_size[0]
        d.tp_size = [d_tp] * count + d.tp_size
        d.dp_size = [d_dp] * count + d.dp_size
        s.tp_size = s.tp_size[:-count]
        s.dp_size = s.dp_size[:-count]
        d.algo = s.algo[-count:] + d.algo
        s.algo = s.algo[:-count]
        nb = src + 1
    elif src > towards:
        d = new.stages[src - 1]
        d.ops = d.ops + s.ops[:count]
        d.recompute_ops = d.recompute_ops + [0] * count
        s.ops = s.ops[count:]
        s.recompute_ops = s.recompute_ops[count:]
        d_tp, d_dp = d.tp_size[-1], d.dp_size[-1]
        d.tp_size = d.tp_size + [d_tp] * count
        d.dp_size = d.dp_size + [d_dp] * count
        s.tp_size = s.tp_size[count:]
        s.dp_size = s.dp_size[count:]
        d.algo = d.algo + s.algo[:count]
        s.algo = s.algo[count:]
        nb = src - 1
    else:
        return plan
    if src_recompute is not None:
        s.recompute_ops = src_recompute
    else:
        ctx.cost.refresh_recompute(new, src)
    ctx.cost.refresh_recompute(new, nb)
    ctx.move_memo[memo_key] = new.clone()
    return new


def _delta_time(ctx, plan, long_stage, short_stage, n_moved, decrease=True):
    """Time of only the ops that would move (used with --predict-delta-time)."""
    s = plan.stages[long_stage]
    ops, rc, tp, dp, algo = s.ops, s.recompute_ops, s.tp_size, s.dp_size, s.algo
    n = len(ops)
    right = long_stage < short_stage
    if right:
        sl = slice(n - n_moved, n)
    else:
        sl = slice(0, n_moved)
    ops_m, algo_m = ops[sl], algo[sl]
    if decrease:
        rc_m, tp_m, dp_m = list(rc[sl]), tp[sl], dp[sl]
    else:
        nb = plan.stages[long_stage + 1] if right else plan.stages[long_stage - 1]
        rc_m = [0] * n_moved
        tp_m = [nb.tp_size[0] if right else nb.tp_size[-1]] * n_moved
        dp_m = [nb.dp_size[0] if right else nb.dp_size[-1]] * n_moved
    mbs = [plan.micro_bs // dp_m[j] for j in range(len(ops_m))]
    fwd, bwd, cin, cout, _ = ctx.cost.stage_time_terms(ops_m, mbs, tp_m, algo_m, dp_m, False, False)
    rct = ctx.cost.recompute_time(ops_m, rc_m, mbs, tp_m, algo_m)
    if right == decrease:
        total = fwd + bwd - cin + cout + rct
    else:
        total = fwd + bwd + cin - cout + rct
    return total / 1000


def prim_migrate_ops(ctx: SearchContext, plan: Plan, bottleneck, action=""):
    args = ctx.args
    metric = "memory" if max(plan.memory_list) > args.memory_limit else "time_with_efficiency"
    partners = [pick_partner_stage(ctx, plan, "mig_workloads", "", bottleneck, metric)
                for _ in range(args.num_partners_in_op_mig)]
    success = time_up = False
    delta_mode = args.predict_delta_time and metric == "time_with_efficiency"
    if delta_mode:
        running = plan.compute_time_list
    for step in range(args.max_op_move_steps):
        step_ok = False
        origin = bottleneck
        for partner in partners:
            if bottleneck is None or partner is None:
                break
            for goal in _migration_goals(ctx, plan, bottleneck, partner, metric):
                bottleneck = origin
                cand = plan.clone()
                while bottleneck != partner:
                    found = False
                    for k in range(0, len(cand.stages[bottleneck].ops), args.op_group_size):
                        if ctx.trial_time_up():
                            time_up = True
                            break
                        if delta_mode:
                            value, rc = running[bottleneck] - _delta_time(ctx, cand, bottleneck, partner, k), None
                        else:
                            value, rc = ctx.cost.value_after_move(cand, bottleneck, partner, k, metric)
                        if value < goal:
                            cand = move_ops_once(ctx, cand, bottleneck, partner, k, rc)
                            found = True
                            running = [ctx.cost.stage_time_cached(cand, i) for i in range(cand.num_stages)]
                            break
                    if time_up:
                        break
                    if found:
                        bottleneck += 1 if bottleneck < partner else -1
                    else:
                        break
                ctx.explored += 1
                if delta_mode:
                    value = running[bottleneck]
                else:
                    value, _ = ctx.cost.value_after_move(cand, bottleneck, bottleneck, 0, metric)
                if value < goal:
                    plan = cand
                    ctx.cost.evaluate(plan)
                    step_ok = success = True
                    break
                if time_up:
                    break
            if step_ok or time_up:
                break
        if not step_ok or time_up:
            break
        bottleneck = pick_target_stage(ctx, plan, metric=metric, tag="mig" + str(step))
        partners = [pick_partner_stage(ctx, plan, "mig_workloads", "", bottleneck, metric, tag="mig" + str(step))
                    for _ in range(args.num_partners_in_op_mig)]
    return plan if success else None


def prim_migrate_ops_simple(ctx: SearchContext, plan: Plan, bottleneck, action=""):
    """One migration step only."""
    args = ctx.args
    metric = "memory" if max(plan.memory_list) > args.memory_limit else "time_with_efficiency"
    partners = [pick_partner_stage(ctx, plan, "mig_workloads", "", bottleneck, metric)
                for _ in range(args.num_partners_in_op_mig)]
    success = time_up = False
    delta_mode = args.predict_delta_time and metric == "time_with_efficiency"
    if delta_mode:
        running = plan.compute_time_list
    for partner in partners:
        if bottleneck is None or partner is None:
            break
        for goal in _migration_goals(ctx, plan, bottleneck, partner, metric):
            cand = plan.clone()
            for k in range(0, len(cand.stages[bottleneck].ops), args.op_group_size):
                if ctx.trial_time_up():
                    time_up = True
                    break
                if delta_mode:
                    value, rc = running[bottleneck] - _delta_time(ctx, cand, bottleneck, partner, k), None
                else:
                    value, rc = ctx.cost.value_after_move(cand, bottleneck, partner, k, metric)
                if value < goal:
                    cand = move_ops_once(ctx, cand, bottleneck, partner, k, rc)
                    success = True
                    running = [ctx.cost.stage_time_cached(cand, i) for i in range(cand.num_stages)]
                    break
            if time_up:
                break
            if success:
                ctx.explored += 1
                plan = cand
                ctx.cost.evaluate(plan)
                break
        if success or time_up:
            break
    return plan if success else None


# ------------------------------------------------------------------------------------------------
# GPU migration between stages (tp / dp degrees)
# ------------------------------------------------------------------------------------------------
def _can_give(ctx, plan, s, dim):
    st = plan.stages[s]
    if st.num_gpus == 1:
        return False
    if dim == "tp" and min(st.tp_size) == 1:
        return False
    if dim == "dp":
        if min(st.dp_size) == 1:
            return False
        for d in st.dp_size:
            if plan.micro_bs // (d // 2) not in ctx.args.micro_batch_size:
                return False
    return True


def _can_take(ctx, plan, s, dim):
    st = plan.stages[s]
    if st.num_gpus * 2 > ctx.args.num_gpus - (plan.num_stages - 1):
        return False
    if dim == "tp" and max(st.tp_size) * 2 > ctx.args.max_tp:
        return False
    if dim == "dp":
        for d in st.dp_size:
            if plan.micro_bs // (d * 2) not in ctx.args.micro_batch_size:
                return False
    return True


def _next_giver(ctx, plan, visited, max_gpus=BIG):
    best_s = best_dim = None
    best_t = BIG
    for s in range(plan.num_stages):
        if s not in visited and plan.stages[s].num_gpus // 2 <= max_gpus:
            for dim in ("tp", "dp"):
                if _can_give(ctx, plan, s, dim):
                    t, _ = ctx.cost.value_after_move(plan, s, None, 0, "time", dec_gpus=True, dim=dim)
                    if t < best_t:
                        best_t, best_s, best_dim = t, s, dim
    return best_s, best_dim


def _next_taker(ctx, plan, visited, max_gpus=BIG):
    best_s = best_dim = None
    best_t = BIG
    for s in range(plan.num_stages):
        if s not in visited and plan.stages[s].num_gpus <= max_gpus:
            for dim in ("tp", "dp"):
                if _can_take(ctx, plan, s, dim):
                    t, _ = ctx.cost.value_after_move(plan, s, None, 0, "time", inc_gpus=True, dim=dim)
                    if t < best_t:
                        best_t, best_s, best_dim = t, s, dim
    return best_s, best_dim


def _scale_degree(plan, s, dim, up: bool):
    st = plan.stages[s]
    if dim == "tp":
        st.tp_size = [x * 2 if up else x // 2 for x in st.tp_size]
    elif dim == "dp":
        st.dp_size = [x * 2 if up else x // 2 for x in st.dp_size]
    else:
        raise RuntimeError(f"unexpected dim {dim}")


def prim_move_gpus(ctx: SearchContext, plan: Plan, bottleneck, action):
    if plan.num_stages <= 1:
        return None
    args = ctx.args
    taker = giver = None
    if "inc" in action:
        taker, taker_dim = bottleneck, action.split("inc_")[1]
        take_n = plan.stages[bottleneck].num_gpus
        if not _can_take(ctx, plan, taker, taker_dim):
            return None
    elif "dec" in action:
        giver, giver_dim = bottleneck, action.split("dec_")[1]
        give_n = plan.stages[bottleneck].num_gpus // 2
        if not _can_give(ctx, plan, giver, giver_dim):
            return None
    best = None
    visited: List[int] = []
    for _ in range(plan.num_stages - 1):
        ctx.explored += 1
        partners: List[int] = []
        if "inc" in action:
            giver, giver_dim = _next_giver(ctx, plan, visited + [bottleneck])
            visited.append(giver)
            if giver is None:
                break
            n_give, n_take = plan.stages[giver].num_gpus // 2, take_n
        else:
            taker, taker_dim = _next_taker(ctx, plan, visited + [bottleneck])
            visited.append(taker)
            if taker is None:
                break
            n_take, n_give = plan.stages[taker].num_gpus, give_n
        new = plan.clone()
        if n_give >= n_take:
            new.stages[giver].num_gpus -= n_give
            _scale_degree(new, giver, giver_dim, up=False)
            if giver != bottleneck:
                partners.append(giver)
            cur_n, cur_s, cur_dim = n_take, taker, taker_dim
            while n_give > 0:
                new.stages[cur_s].num_gpus += cur_n
                _scale_degree(new, cur_s, cur_dim, up=True)
                n_give -= cur_n
                if cur_s != bottleneck:
                    partners.append(cur_s)
                if n_give > 0:
                    cur_s, cur_dim = _next_taker(ctx, plan, partners + [bottleneck], n_give)
                    if cur_s is None:
                        break
                    cur_n = plan.stages[cur_s].num_gpus
        else:
            new.stages[taker].num_gpus += n_take
            _scale_degree(new, taker, taker_dim, up=True)
            if taker != bottleneck:
                partners.append(taker)
            cur_s, cur_n, cur_dim = giver, n_give, giver_dim
            while n_take > 0:
                new.stages[cur_s].num_gpus -= cur_n
                _scale_degree(new, cur_s, cur_dim, up=False)
                n_take -= cur_n
                if cur_s != bottleneck:
                    partners.append(cur_s)
                if n_take > 0:
                    cur_s, cur_dim = _next_giver(ctx, plan, partners + [bottleneck], n_take)
                    if cur_s is None:
                        break
                    cur_n = plan.stages[cur_s].num_gpus // 2
        if is_legal(new, args.num_gpus, args.num_gpus_per_node, args.num_nodes):
            best = new
            break
    if best is not None:
        ctx.cost.refresh_recompute(best)
    return best


# ------------------------------------------------------------------------------------------------
# micro-batch size
# ------------------------------------------------------------------------------------------------
def _neighbour_mbs(mbs, choices, up):
    i = choices.index(mbs)
    if up:
        return choices[i + 1] if i < len(choices) - 1 else mbs
    return choices[i - 1] if i > 0 else mbs


def best_stage_layout(ctx: SearchContext, stage: StagePlan, micro_bs: int, num_gpus: int):
    """Best (tp, dp) with tp * dp = num_gpus for a whole stage by total GPU time, with a memory penalty."""
    if num_gpus == 0:
        return BIG, None
    args, cost = ctx.args, ctx.cost
    best_t = BIG
    best = stage.clone()
    tp = 1
    n = len(stage.ops)
    while tp <= args.max_tp:
        dp = num_gpus // tp
        if dp >= 1 and micro_bs // dp in args.micro_batch_size:
            tps, dps = [tp] * n, [dp] * n
            rc = cost.choose_recompute(stage.ops, micro_bs, tps, dps, stage.num_stages_behind, stage.algo)
            t = cost.stage_time(stage.ops, rc, tps, dps, micro_bs, stage.algo) * num_gpus
            m = cost.stage_memory(stage.ops, rc, tps, dps, micro_bs, stage.num_stages_behind, stage.algo)
            if m > args.memory_limit:
                t += m * 10
            if t < best_t:
                best_t = t
                best.tp_size, best.dp_size, best.num_gpus, best.recompute_ops = tps, dps, num_gpus, rc
        tp *= 2
    return (best_t, best) if best_t < BIG else (best_t, None)


def prim_change_mbs(ctx: SearchContext, plan: Plan, bottleneck, action):
    ctx.explored += 1
    choices = ctx.args.micro_batch_size
    up = action == "inc_mbs"
    if up and not plan.micro_bs < choices[-1]:
        return None
    if not up and not plan.micro_bs > choices[0]:
        return None
    new = plan.clone()
    new.micro_bs = _neighbour_mbs(new.micro_bs, choices, up)
    for i in range(new.num_stages):
        if not ctx.args.simple_prim_mbs:
            _, st = best_stage_layout(ctx, new.stages[i], new.micro_bs, new.stages[i].num_gpus)
            if st is None:
                return None
            new.stages[i] = st
        elif not up:
            if new.micro_bs // max(new.stages[i].dp_size) not in choices:
                return None
    return new


# ------------------------------------------------------------------------------------------------
# fine-tuning passes
# ------------------------------------------------------------------------------------------------
def finetune_stage_layouts(ctx: SearchContext, plan: Plan) -> Plan:
    ctx.explored += 1
    new = plan.clone()
    for i in range(new.num_stages):
        _, st = best_stage_layout(ctx, new.stages[i], plan.micro_bs, new.stages[i].num_gpus)
        if st is not None:
            new.stages[i] = st
    return new


def _retune_run(ctx, plan, s, start, grow, reverse):
    """Flip tp <-> dp for the longest run of ops starting at `start` (forwards or backwards) that allows it."""
    st = plan.stages[s]
    args = ctx.args
    tp, dp, mbs = st.tp_size, st.dp_size, plan.micro_bs
    idxs = range(start, -1, -1) if reverse else range(start, len(st.ops))
    ntp = ndp = None
    for i in idxs:
        if grow == "dp":
            ok = tp[i] > 1 and mbs // (dp[i] * 2) in args.micro_batch_size
        elif grow == "tp":
            ok = tp[i] < args.max_tp and dp[i] > 1 and mbs // (dp[i] // 2) in args.micro_batch_size
        else:
            raise RuntimeError(f"inc dim {grow} not supported.")
        if not ok:
            break
        if ntp is None:
            ntp, ndp = list(tp), list(dp)
            ctx.explored += 1
        if grow == "dp":
            ntp[i] //= 2
            ndp[i] *= 2
        else:
            ntp[i] *= 2
            ndp[i] //= 2
    if ntp is None:
        return None
    rc = ctx.cost.choose_recompute(st.ops, mbs, ntp, ndp, st.num_stages_behind, st.algo)
    t = ctx.cost.stage_time(st.ops, rc, ntp, ndp, mbs, st.algo)
    m = ctx.cost.stage_memory(st.ops, rc, ntp, ndp, mbs, st.num_stages_behind, st.algo)
    return ntp, ndp, rc, t, m


def finetune_op_degrees(ctx: SearchContext, plan: Plan, s: int, goal="time") -> Optional[Plan]:
    st = plan.stages[s]
    if st.num_gpus == 1:
        return None
    cands = []
    for start in range(len(st.ops)):
        if st.ops[start] in ctx.tunable:
            for grow in ("tp", "dp"):
                for reverse in (False, True):
                    r = _retune_run(ctx, plan, s, start, grow, reverse)
                    if r is not None:
                        cands.append(r)
    if not cands:
        return None
    limit = ctx.args.memory_limit
    pick = 0
    if goal == "time" and min(c[4] for c in cands) < limit:
        best = BIG
        for i, c in enumerate(cands):
            if c[4] < limit and c[3] < best:
                best, pick = c[3], i
    else:
        best = BIG
        for i, c in enumerate(cands):
            if c[4] < best:
                best, pick = c[4], i
    new = plan.clone()
    new.stages[s].tp_size, new.stages[s].dp_size, new.stages[s].recompute_ops = cands[pick][0], cands[pick][1], cands[pick][2]
    return new


def finetune_op_algos(ctx: SearchContext, plan: Plan, s: int) -> Optional[Plan]:
    st = plan.stages[s]
    if st.num_gpus == 1:
        return None
    cost, limit = ctx.cost, ctx.args.memory_limit
    ops, rc, tp, dp, mbs, behind = st.ops, st.recompute_ops, st.tp_size, st.dp_size, plan.micro_bs, st.num_stages_behind
    algo = st.algo
    prev_t = cost.stage_time(ops, rc, tp, dp, mbs, algo)
    prev_m = cost.stage_memory(ops, rc, tp, dp, mbs, behind, algo)
    changed = False
    for i in range(len(ops)):
        if ops[i] not in ctx.tunable:
            continue
        trials = []
        for a in range(ctx.args.num_algos):
            if a != algo[i]:
                ctx.explored += 1
                cand = list(algo)
                cand[i] = a
                trials.append((cost.stage_time(ops, rc, tp, dp, mbs, cand),
                               cost.stage_memory(ops, rc, tp, dp, mbs, behind, cand), cand))
        pick = -1
        if prev_m > limit:
            best = BIG
            for j, (t, m, _) in enumerate(trials):
                if t < best:
                    best, pick = t, j
        else:
            best = prev_t
            for j, (t, m, _) in enumerate(trials):
                if t < best and m < limit:
                    best, pick = t, j
        if pick >= 0:
            changed = True
            prev_t, prev_m, algo = trials[pick]
    if not changed:
        return None
    new = plan.clone()
    new.stages[s].algo = algo
    return new


def finetune(ctx: SearchContext, plan: Plan) -> Plan:
    limit = ctx.args.memory_limit
    for s in range(plan.num_stages):
        t0 = plan.time_list[s]
        cand = finetune_op_degrees(ctx, plan, s)
        if cand is not None:
            ctx.cost.evaluate(cand)
            if cand.time_list[s] < t0 and cand.memory_list[s] <= limit:
                plan, t0 = cand, cand.time_list[s]
        cand = finetune_op_algos(ctx, plan, s)
        if cand is not None:
            ctx.cost.evaluate(cand)
            if cand.time_list[s] < t0 and cand.memory_list[s] <= limit:
                plan = cand
    return plan


def prim_exchange_degrees(ctx: SearchContext, plan: Plan, s, action):
    ctx.explored += 1
    st = plan.stages[s]
    new = None
    if action == "inc_tp_dec_dp" and min(st.dp_size) > 1 and max(st.tp_size) * 2 <= ctx.args.max_tp:
        new = plan.clone()
        new.stages[s].tp_size = [x * 2 for x in new.stages[s].tp_size]
        new.stages[s].dp_size = [x // 2 for x in new.stages[s].dp_size]
    elif action == "inc_dp_dec_tp" and min(st.tp_size) > 1:
        for d in st.dp_size:
            if plan.micro_bs // (d * 2) not in ctx.args.micro_batch_size:
                return None
        new = plan.clone()
        new.stages[s].dp_size = [x * 2 for x in new.stages[s].dp_size]
        new.stages[s].tp_size = [x // 2 for x in new.stages[s].tp_size]
    if new is not None:
        ctx.cost.refresh_recompute(new)
    return new


def action_table(ctx: SearchContext) -> List[Primitive]:
    mig = prim_migrate_ops_simple if ctx.args.simple_prim_mig else prim_migrate_ops
    table = [
        Primitive("dec_op", "-", "-", "0", "-", "0", "0", mig),
        Primitive("inc_dp", "-", "-", "+", "0", "-", "+", prim_move_gpus),
        Primitive("dec_dp", "+", "+", "-", "0", "+", "-", prim_move_gpus),
        Primitive("inc_tp", "-", "-", "+", "0", "-", "+", prim_move_gpus),
        Primitive("dec_tp", "+", "+", "-", "0", "+", "-", prim_move_gpus),
        Primitive("inc_mbs", "-", "+", "0", "0", "+", "0", prim_change_mbs),
        Primitive("dec_mbs", "+", "-", "0", "0", "-", "0", prim_change_mbs),
    ]
    if ctx.args.add_action_tp_dp_exchange:
        table += [Primitive("inc_tp_dec_dp", "+", "-", "0", "0", "-", "+", prim_exchange_degrees),
                  Primitive("inc_dp_dec_tp", "-", "+", "0", "0", "+", "-", prim_exchange_degrees)]
    return table
