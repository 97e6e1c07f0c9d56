"""Cost model: predicts per-stage time and memory of a plan from the profiled database.

Reproduces the reference model term by term (search/aceso_cost_model.py) -- the arithmetic order is kept
so that predictions on the reference's committed databases are bit-identical -- and extends it with one
optional term: when a database carries the columns `fwd_overlap_comm` / `bwd_overlap_comm` (communication time
hidden behind an op's own compute), they are subtracted from the op's time.  This framework's op profiler times a
tensor-parallel op WITH its fused collective inside the timed region, so its tables already hold the overlapped time
and it writes zeros in those columns; they serve databases measured with unfused collectives.  Databases without
the columns predict as before.

  stage time      = (sum fwd + sum bwd + boundary-in comm + boundary-out comm + recompute fwd) / 1000  [ms]
  pipeline time_i = stage_time_i * (num_microbatches - 1) + sum_j stage_time_j
  stage memory    = weights * (1 + main params) + grads + optimizer
                    + (inputs + activations - saved by recompute) * stages_behind + peak + reserved
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

from .config import Plan
from .database import ProfileDB
from .opinfo import op_spec, reshard_primitives


@dataclass
class CostOptions:
    memory_limit: float = 28000
    num_gpus_per_node: int = 8
    main_params_factor: float = 2       # fp32 master copy, in units of the weight bytes
    optimizer_factor: float = 4
    resharding: bool = True
    consider_shared_space: bool = True
    consider_reserved_space: bool = True
    consider_collective_memory: bool = False
    support_comm_predict: bool = False
    memory_pred_type: str = "MAX"
    flex_recompute: bool = True
    peak_mem_in_backward: float = 0
    price_overlap: bool = True
    never_recompute: Sequence[str] = ()


_SHARED_ZERO = ("enc-attention-softmax", "bn1")


def _shares_buffer(op: str) -> bool:
    """Ops whose saved activation aliases a neighbour's (softmax / in-place BN / downsample add)."""
    return op in _SHARED_ZERO or "-bn3" in op or ("-downsample" in op and "0-0" not in op)


try:  # built by `python -m superscaler_b200.build`; the Python definitions below are the same arithmetic
    from .. import _search_native as _native
except ImportError:  # pragma: no cover
    _native = None


class CostModel:
    def __init__(self, db: ProfileDB, opt: CostOptions):
        self.db, self.opt = db, opt
        self._mem_cache: Dict[tuple, float] = {}
        self._time_cache: Dict[tuple, float] = {}
        t = db.table
        self._fwd, self._bwd, self._in, self._out = t["fwd"], t["bwd"], t["in_mb"], t["out_mb"]
        self._w, self._a, self._rf, self._rb = t["weights"], t["acts"], t["res_fwd"], t["res_bwd"]
        self._fo, self._bo = t["fwd_ovl"], t["bwd_ovl"]
        self._mi = db.mbs_index
        self._overlap = opt.price_overlap and db.has_overlap_columns
        # per-name facts and the tp -> table index map, computed once (the search calls these millions of times)
        self._lg = {1 << k: int(math.log(1 << k, 2)) for k in range(16)}
        self._name_ids: Dict[tuple, int] = {}
        self._groups_cache: Dict[int, tuple] = {}
        self._stage_time_cache: Dict[tuple, float] = {}
        self._rc_cache: Dict[tuple, tuple] = {}
        self._arrays_cache: Dict[tuple, tuple] = {}
        self._names_cache: Dict[tuple, tuple] = {}
        self._terms_cache: Dict[tuple, tuple] = {}
        self._exact_mem_cache: Dict[tuple, object] = {}
        self._kind: Dict[str, int] = {}          # 0 plain, 1 counted 1.5x (attention dropout), 2 aliases a neighbour
        self._starts_layer: Dict[str, bool] = {}

    # ---- memo keys ---------------------------------------------------------------------------
    def _nid(self, ops) -> int:
        """Small integer standing for the exact sequence of op names (memo keys hash it instead of the names)."""
        names = tuple(ops)
        i = self._name_ids.get(names)
        if i is None:
            i = self._name_ids[names] = len(self._name_ids)
        return i

    @staticmethod
    def _ck(seq):
        """Per-op list as a memo key part: the value itself when all entries are equal (the usual case), else a tuple."""
        v = seq[0]
        return v if seq.count(v) == len(seq) else tuple(seq)

    # ---- time -------------------------------------------------------------------------------
    def stage_time_terms(self, ops, mbs, tp, algo, dp, in_cross_node, out_cross_node):
        """(fwd us, bwd us, boundary-in us, boundary-out us, tp/reshard comm us).  Memoised on its exact
        arguments: the search prices the same stage slice many times."""
        if len(ops) == 0:
            return 0, 0, 0, 0, 0
        ck = self._ck
        key = (self._nid(ops), ck(mbs), ck(tp), ck(algo), ck(dp), in_cross_node, out_cross_node)
        hit = self._terms_cache.get(key)
        if hit is None:
            if len(self._terms_cache) > 50000:
                self._terms_cache.clear()
            hit = self._terms_cache[key] = self._stage_time_terms(ops, mbs, tp, algo, dp, in_cross_node,
                                                                  out_cross_node)
        return hit

    def _stage_time_terms(self, ops, mbs, tp, algo, dp, in_cross_node, out_cross_node):
        mi, db = self._mi, self.db
        fwd = bwd = 0
        tp_comm = 0
        lg = self._lg
        for i in range(len(ops)):
            op = ops[i]
            a, b, c = mi[mbs[i]], lg[tp[i]], algo[i]
            fwd += self._fwd[op][a][b][c]
            bwd += self._bwd[op][a][b][c]
            if self._overlap:
                fwd -= self._fo[op][a][b][c]
                bwd -= self._bo[op][a][b][c]
            if self.opt.support_comm_predict:
                for suffix in ("qkv", "dense", "GEMM", "conv", "downsample"):
                    if suffix in op:
                        tp_comm += db.collective_time("all_reduce", tp[i], self._out[op][a][b][c]) * 1000
        in_size = self._in[ops[0]][mi[mbs[0]]][lg[tp[0]]][algo[0]]
        out_size = self._out[ops[-1]][mi[mbs[-1]]][lg[tp[0]]][algo[-1]]
        in_comm = in_size / (db.inter_bandwidth(in_size) if in_cross_node else db.intra_bandwidth(in_size))
        out_comm = out_size / (db.inter_bandwidth(out_size) if out_cross_node else db.intra_bandwidth(out_size))
        fwd_rs = bwd_rs = 0
        if self.opt.resharding:
            for i in range(1, len(ops)):
                if tp[i] == tp[i - 1] and dp[i] == dp[i - 1] and algo[i] == algo[i - 1] and tp[i] == 1:
                    continue  # single-device layouts are always identical
                src = op_spec(ops[i - 1], tp[i - 1], dp[i - 1], algo[i - 1], as_input=False)
                dst = op_spec(ops[i], tp[i], dp[i], algo[i], as_input=True)
                f, b, n = reshard_primitives(src, dst)
                if f is None and b is None:
                    continue
                size = self._in[ops[i]][mi[mbs[i]]][lg[tp[i]]][algo[i]]
                if f is not None:
                    fwd_rs += db.collective_time(f, n, size)
                if b is not None:
                    bwd_rs += db.collective_time(b, n, size)
        in_comm += fwd_rs * 1000
        out_comm += bwd_rs * 1000
        tp_comm += fwd_rs * 1000 + bwd_rs * 1000
        return fwd, bwd, in_comm, out_comm, tp_comm

    def recompute_time(self, ops, recompute, mbs, tp, algo):
        if len(ops) == 0 or sum(recompute) == 0:
            return 0
        total = 0
        fwd, mi, lg = self._fwd, self._mi, self._lg
        for i in range(len(ops)):
            if recompute[i] == 1:
                total += fwd[ops[i]][mi[mbs[i]]][lg[tp[i]]][algo[i]]
        return total

    def stage_time(self, ops, recompute, tp, dp, micro_bs, algo) -> float:
        if len(ops) == 0:
            return self._stage_time(ops, recompute, tp, dp, micro_bs, algo)
        ck = self._ck
        key = (self._nid(ops), bytes(recompute), ck(tp), ck(dp), micro_bs, ck(algo))
        hit = self._stage_time_cache.get(key)
        if hit is None:
            if len(self._stage_time_cache) > 100000:
                self._stage_time_cache.clear()
            hit = self._stage_time_cache[key] = self._stage_time(ops, recompute, tp, dp, micro_bs, algo)
        return hit

    def _stage_time(self, ops, recompute, tp, dp, micro_bs, algo) -> float:
        mbs = [micro_bs // dp[j] for j in range(len(ops))]
        fwd, bwd, cin, cout, _ = self.stage_time_terms(ops, mbs, tp, algo, dp, False, False)
        rc = self.recompute_time(ops, recompute, mbs, tp, algo)
        return (fwd + bwd + cin + cout + rc) / 1000

    def stage_time_cached(self, plan: Plan, s: int) -> float:
        st = plan.stages[s]
        key = (st.ops[0], len(st.ops), tuple(st.tp_size), tuple(st.dp_size), tuple(st.recompute_ops),
               tuple(st.algo), plan.micro_bs)
        v = self._time_cache.get(key)
        if v is None:
            v = self.stage_time(st.ops, st.recompute_ops, st.tp_size, st.dp_size, plan.micro_bs, st.algo)
            self._time_cache[key] = v
        return v

    # ---- memory -----------------------------------------------------------------------------
    def _act(self, op, mbs, tp, algo):
        return self._a[op][self._mi[mbs]][self._lg[tp]][algo]

    def _act_arrays(self, ops, mbs, tp, algo):
        """Per op of a stage: its activation size, its accounting kind (see _kind) and whether the NEXT op starts a
        layer (recompute segments end there).  The three passes below walk these lists instead of the tables."""
        names = tuple(ops)
        ck = self._ck
        key = (self._nid(names), ck(mbs), ck(tp), ck(algo))
        hit = self._arrays_cache.get(key)
        if hit is not None:
            return hit
        by_name = self._names_cache.get(names)
        if by_name is None:
            kind_of, starts = self._kind, self._starts_layer
            for op in set(names):
                if op not in kind_of:
                    kind_of[op] = 1 if op == "enc-attention-dropout" else (2 if _shares_buffer(op) else 0)
                    starts[op] = op in ("enc-1st-layernorm",) or "-conv1" in op
            kinds = [kind_of[op] for op in names] if self.opt.consider_shared_space else [0] * len(names)
            ends = [starts[op] for op in names[1:]]
            if len(self._names_cache) > 20000:
                self._names_cache.clear()
            by_name = self._names_cache[names] = (kinds, ends)
        kinds, ends = by_name
        a, mi, lg = self._a, self._mi, self._lg
        n = len(names)
        if tp.count(tp[0]) == n and mbs.count(mbs[0]) == n and algo.count(algo[0]) == n:
            i1, i2, i3 = mi[mbs[0]], lg[tp[0]], algo[0]
            acts = [a[op][i1][i2][i3] for op in names]
        else:
            acts = [a[op][mi[m]][lg[t]][g] for op, m, t, g in zip(names, mbs, tp, algo)]
        if len(self._arrays_cache) > 20000:
            self._arrays_cache.clear()
        out = self._arrays_cache[key] = (acts, kinds, ends)
        return out

    @staticmethod
    def _saved_fast(recompute, acts, kinds, ends):
        n = len(acts)
        if n <= 1 or sum(recompute) == 0:
            return 0
        if _native is not None:
            return _native.saved_by_recompute(recompute, acts, kinds, ends)
        saved = 0
        for i in range(n - 1):
            if recompute[i] == 1 and recompute[i + 1] == 1:
                k = kinds[i]
                if k == 1:
                    saved += acts[i] * 1.5
                elif k == 0 and not ends[i]:
                    saved += acts[i]
        return saved

    @staticmethod
    def _peak_fast(recompute, acts, kinds, ends):
        n = len(acts)
        if n <= 1 or sum(recompute) == 0:
            return 0
        if _native is not None:
            return _native.peak_recompute(recompute, acts, kinds, ends)
        run = 0
        best = 0
        last = n - 1
        for i in range(last):
            if recompute[i] == 1 and recompute[i + 1] == 1:
                k = kinds[i]
                if k == 1:
                    run += acts[i] * 1.5
                elif k == 0:
                    run += acts[i]
                    if ends[i] or i + 1 == last:
                        if run > best:
                            best = run
                        run = 0
            elif run > 0:
                if run > best:
                    best = run
                run = 0
        return best

    def activation_size(self, op, mbs, tp, algo=0):
        return self._act(op, mbs, tp, algo)

    def _memory_terms(self, ops, mbs, tp, algo, arrays=None):
        inputs = self._in[ops[0]][self._mi[mbs[0]]][self._lg[tp[0]]][algo[0]]
        act_of, kinds, _ = arrays if arrays is not None else self._act_arrays(ops, mbs, tp, algo)
        acts = 0
        weights = 0
        w, mi, lg = self._w, self._mi, self._lg
        for i in range(len(ops)):
            k = kinds[i]
            if k == 1:
                acts += act_of[i] * 1.5
            elif k == 0:
                acts += act_of[i]
            weights += w[ops[i]][mi[mbs[i]]][lg[tp[i]]][algo[i]]
        return weights, inputs, acts

    def _reserved(self, ops, mbs, tp, dp, algo, weight_mb):
        rf = rb = 0
        for i in range(len(ops) - 1):
            a, b, c = self._mi[mbs[i]], self._lg[tp[i]], algo[i]
            v = self._rf[ops[i]][a][b][c]
            if v > rf:
                rf = v
            v = self._rb[ops[i]][a][b][c]
            if v > rb:
                rb = v
        coll = 0
        if self.opt.consider_collective_memory and self.opt.resharding:
            for i in range(1, len(ops)):
                src = op_spec(ops[i - 1], tp[i - 1], dp[i - 1], algo[i - 1], as_input=False)
                dst = op_spec(ops[i], tp[i], dp[i], algo[i], as_input=True)
                f, b, n = reshard_primitives(src, dst)
                size = self._in[ops[i]][self._mi[mbs[i]]][self._lg[tp[i]]][algo[i]]
                for prim in (f, b):
                    if prim is not None:
                        m = size * n if prim in ("all_gather", "all_to_all") else size
                        if m > coll:
                            coll = m
        if self.opt.memory_pred_type == "MAX":
            return max(rf + rb, weight_mb) + coll
        if self.opt.memory_pred_type == "MIN":
            return max(rf, rb, weight_mb, coll)
        raise RuntimeError(f"unknown memory_pred_type {self.opt.memory_pred_type}")

    def stage_memory(self, ops, recompute, tp, dp, micro_bs, stages_behind, algo, breakdown=False):
        ck = self._ck
        key = (self._nid(ops), bytes(recompute), ck(tp), ck(dp), micro_bs, stages_behind, ck(algo), breakdown)
        hit = self._exact_mem_cache.get(key)
        if hit is None:
            if len(self._exact_mem_cache) > 50000:
                self._exact_mem_cache.clear()
            hit = self._exact_mem_cache[key] = self._stage_memory(ops, recompute, tp, dp, micro_bs, stages_behind,
                                                                  algo, breakdown)
        return hit

    def _stage_memory(self, ops, recompute, tp, dp, micro_bs, stages_behind, algo, breakdown=False):
        mbs = [micro_bs // dp[j] for j in range(len(ops))]
        arrays = self._act_arrays(ops, mbs, tp, algo)
        w, inputs, acts = self._memory_terms(ops, mbs, tp, algo, arrays)
        grads = w
        main = w * self.opt.main_params_factor
        optim = w * self.opt.optimizer_factor
        saved = self._saved_fast(recompute, *arrays)
        peak_rc = self._peak_fast(recompute, *arrays)
        reserved = self._reserved(ops, mbs, tp, dp, algo, w) if self.opt.consider_reserved_space else 0
        in_flight = (inputs + acts - saved) * stages_behind
        peak = inputs + acts - saved + peak_rc
        w += main
        if breakdown:
            return w, grads, optim, in_flight, peak, reserved
        return w + grads + optim + in_flight + peak + reserved

    def stage_memory_cached(self, ops, recompute, tp, dp, micro_bs, stages_behind, algo) -> float:
        key = (ops[0], len(ops), tuple(tp), tuple(dp), tuple(recompute), tuple(algo), micro_bs, stages_behind)
        v = self._mem_cache.get(key)
        if v is None:
            v = self.stage_memory(ops, recompute, tp, dp, micro_bs, stages_behind, algo)
            self._mem_cache[key] = v
        return v

    def reserved_list(self, plan: Optional[Plan]) -> List[float]:
        if plan is None:
            return []
        return [self.stage_memory(s.ops, s.recompute_ops, s.tp_size, s.dp_size, plan.micro_bs, s.num_stages_behind,
                                  s.algo, breakdown=True)[5] for s in plan.stages]

    # ---- recompute selection ----------------------------------------------------------------
    def choose_recompute(self, ops, micro_bs, tp, dp, stages_behind, algo) -> List[int]:
        """Greedy: while the stage exceeds the memory limit, recompute the op kind that frees the most
        activation memory (together with the op that follows it)."""
        n = len(ops)
        if not self.opt.flex_recompute:
            return [1] * n
        # the search asks the same question again and again (the same candidate move from many trials): the answer
        # depends on nothing but these arguments
        ck = self._ck
        key = (self._nid(ops), micro_bs, ck(tp), ck(dp), stages_behind, ck(algo))
        hit = self._rc_cache.get(key)
        if hit is not None:
            return list(hit)
        rc = self._choose_recompute(ops, micro_bs, tp, dp, stages_behind, algo)
        if len(self._rc_cache) > 50000:
            self._rc_cache.clear()
        self._rc_cache[key] = tuple(rc)
        return rc

    def _choose_recompute(self, ops, micro_bs, tp, dp, stages_behind, algo) -> List[int]:
        n = len(ops)
        rc = [0] * n
        mem = self.stage_memory_cached(ops, rc, tp, dp, micro_bs, stages_behind, algo) + self.opt.peak_mem_in_backward
        limit = self.opt.memory_limit
        if mem - limit <= 0:
            return rc
        mbs = [micro_bs // dp[i] for i in range(len(dp))]
        acts, kinds, ends = self._act_arrays(ops, mbs, tp, algo)
        never = self.opt.never_recompute
        if _native is not None:
            nid = self._nid(ops)
            grouping = self._groups_cache.get(nid)
            if grouping is None:
                ids: Dict[str, int] = {}
                group_of = [ids.setdefault(op, len(ids)) for op in ops]
                eligible = [int(name not in ("enc-1st-layernorm",) and "-conv1" not in name and "-relu" not in name
                                and name not in never) for name in ids]
                grouping = self._groups_cache[nid] = (group_of, eligible)
            return _native.choose_recompute(acts, kinds, ends, grouping[0], grouping[1], mem, limit, stages_behind)
        groups: Dict[str, dict] = {}
        for i in range(n):
            g = groups.setdefault(ops[i], {"index": [], "size": [], "done": False, "sum": 0})
            sz = acts[i] * (stages_behind + 1)
            g["index"].append(i)
            g["size"].append(sz)
            g["sum"] += sz
        saved0 = 0
        peak0 = self._peak_fast(rc, acts, kinds, ends)
        while mem - limit > 0:
            # pick the not-yet-recomputed op kind with the largest total activation
            best, best_sz = None, 0
            for name, g in groups.items():
                if not g["done"] and g["sum"] > best_sz and name not in ("enc-1st-layernorm",) \
                        and "-conv1" not in name and "-relu" not in name and name not in never:
                    best, best_sz = name, g["sum"]
            if best_sz == 0:
                break
            g = groups[best]
            g["done"] = True
            nxt = g["index"][0] + 1
            if nxt >= n:
                break
            groups[ops[nxt]]["done"] = True
            exceed = mem - limit
            if best_sz < exceed:
                idxs = g["index"]
            else:
                acc, k = 0, 0
                while acc <= exceed and k < len(g["size"]):
                    acc += g["size"][k]
                    k += 1
                idxs = list(g["index"][:k])
            for i in idxs:
                if i >= 0:
                    rc[i] = 1
                    if i < n - 1:
                        rc[i + 1] = 1
                else:
                    break
            saved1 = self._saved_fast(rc, acts, kinds, ends)
            mem -= (saved1 - saved0) * (stages_behind + 1)
            saved0 = saved1
            peak1 = self._peak_fast(rc, acts, kinds, ends)
            mem += peak1 - peak0
            peak0 = peak1
        return rc

    def refresh_recompute(self, plan: Plan, stage: Optional[int] = None) -> None:
        for i in ([stage] if stage is not None else range(plan.num_stages)):
            s = plan.stages[i]
            s.recompute_ops = self.choose_recompute(s.ops, plan.micro_bs, s.tp_size, s.dp_size, s.num_stages_behind,
                                                    s.algo)

    # ---- whole-plan evaluation --------------------------------------------------------------
    def evaluate(self, plan: Plan, report: Optional[list] = None) -> None:
        """Fills the plan's time / memory lists and the per-GPU breakdown the policy reads."""
        micro_bs = plan.micro_bs
        nb = plan.global_bs // micro_bs
        per_node = self.opt.num_gpus_per_node
        raw, mem, comp, eff, gpu_t, ideal_l, loss_l, rc_l = [], [], [], [], [], [], [], []
        seen = 0
        for i, s in enumerate(plan.stages):
            ops, g = s.ops, s.num_gpus
            mbs = [micro_bs // s.dp_size[j] for j in range(len(ops))]
            in_x = (seen % per_node) == 0 and seen > 0
            seen += g
            out_x = (seen % per_node) == 0
            fwd, bwd, cin, cout, tpc = self.stage_time_terms(ops, mbs, s.tp_size, s.algo, s.dp_size, in_x, out_x)
            rc = self.recompute_time(ops, s.recompute_ops, mbs, s.tp_size, s.algo)
            t = (fwd + bwd + cin + cout + rc) / 1000
            raw.append(t)
            comp.append((fwd + bwd + rc) / 1000)
            gpu_t.append(t * g)
            one = [1] * len(ops)
            f1, b1, ci1, co1, _ = self.stage_time_terms(ops, [micro_bs] * len(ops), one, s.algo, one, in_x, out_x)
            ideal = (f1 + b1 + ci1 + co1) / 1000
            loss = (fwd + bwd) - (f1 + b1) / g
            ideal_l.append(((f1 + b1) / g) / 1000)
            loss_l.append(loss / 1000)
            rc_l.append(rc / 1000)
            parts = self.stage_memory(ops, s.recompute_ops, s.tp_size, s.dp_size, micro_bs, s.num_stages_behind,
                                      s.algo, breakdown=True)
            w, gr, op_, infl, peak, res = parts
            mem.append(w + gr + op_ + infl + peak + res)
            eff.append(ideal / (t * g))
            if report is not None:
                report.append({"stage": i, "fwd_ms": fwd / 1000 * nb, "bwd_ms": (bwd + rc) / 1000 * nb,
                               "recompute_ms": rc / 1000 * nb, "in_comm_ms": cin / 1000 * nb,
                               "out_comm_ms": cout / 1000 * nb, "reshard_ms": tpc / 1000 * nb, "weights_mb": w,
                               "grads_mb": gr, "optimizer_mb": op_, "activations_mb": infl, "peak_mb": peak,
                               "reserved_mb": res})
        total = sum(raw)
        times = [raw[i] * (nb - 1) + total for i in range(plan.num_stages)]
        plan.time_list = times
        plan.memory_list = mem
        plan.compute_time_list = comp
        plan.total_gpu_time = sum(gpu_t) * (nb - 1)
        plan.ideal_time_per_gpu = ideal_l
        plan.eff_loss_time_per_gpu = loss_l
        plan.recomp_time_per_gpu = rc_l
        tmax = max(times)
        limit = self.opt.memory_limit
        idle_eff = []
        for i, s in enumerate(plan.stages):
            used_t, used_m = times[i], mem[i]
            if sum(s.recompute_ops) > 0:
                idle = (tmax - used_t) / 2
            else:
                by_time = tmax - used_t
                by_mem = ((limit - used_m) / used_m) * used_t
                idle = by_time if by_mem > by_time else by_mem + (by_time - by_mem) / 2
            idle_eff.append(idle * s.num_gpus * eff[i])
        plan.efficient_time_list = idle_eff
        if report is not None:
            for i, r in enumerate(report):
                r["pipeline_time_ms"] = times[i]
                r["memory_mb"] = mem[i]

    # ---- what-if for op migration -----------------------------------------------------------
    def value_after_move(self, plan: Plan, stage: int, partner, n_moved: int, metric: str, inc_gpus=False,
                         dec_gpus=False, dim=None):
        """Predicted time (ms) or memory (MB) of `stage` after moving `n_moved` ops towards `partner` and/or
        doubling / halving its tp or dp; also returns the recompute flags that go with it."""
        s = plan.stages[stage]
        ops, tp, dp, algo, rc = list(s.ops), list(s.tp_size), list(s.dp_size), list(s.algo), list(s.recompute_ops)
        if n_moved > 0:
            if stage < partner:
                ops, tp, dp, algo = ops[:-n_moved], tp[:-n_moved], dp[:-n_moved], algo[:-n_moved]
            else:
                ops, tp, dp, algo = ops[n_moved:], tp[n_moved:], dp[n_moved:], algo[n_moved:]
        if inc_gpus:
            if dim == "tp":
                tp = [x * 2 for x in tp]
            elif dim == "dp":
                dp = [x * 2 for x in dp]
        if dec_gpus:
            if dim == "tp":
                tp = [x // 2 for x in tp]
            elif dim == "dp":
                dp = [x // 2 for x in dp]
        if n_moved > 0 or inc_gpus or dec_gpus:
            rc = self.choose_recompute(ops, plan.micro_bs, tp, dp, s.num_stages_behind, algo)
        if metric in ("time", "time_with_efficiency"):
            return self.stage_time(ops, rc, tp, dp, plan.micro_bs, algo), rc
        if metric == "memory":
            return self.stage_memory(ops, rc, tp, dp, plan.micro_bs, s.num_stages_behind, algo), rc
        raise RuntimeError(f"metric {metric} not implemented.")
