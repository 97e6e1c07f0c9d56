"""Longer fuzz runs of the plan space than the test suite affords (not collected by pytest):

    python tests/fuzz_plans.py --first-seed 0 --seeds 20 [--kinds layouts cuts interleaved t5 bert]

Every seed draws random plans (per-op layouts + algorithms + recompute flags on two ranks; pipeline cuts with random
GPU counts on four ranks; interleaved plans with random virtual-stage cuts; T5 cuts; BERT layouts and cuts on a padded batch) and trains them on gloo ranks
against the single-process run, with the workers and tolerances of tests/test_parallel_cpu.py and
tests/test_interleaved_cpu.py.  Prints one line per (kind, seed); exit code 1 if any failed.
"""
import argparse
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import test_interleaved_cpu as IL  # noqa: E402
import test_parallel_cpu as PP  # noqa: E402
from dist_utils import run_ranks  # noqa: E402
from helpers import tiny_gpt_plan, tiny_t5_plan  # noqa: E402
from superscaler_b200.runtime.schedules import interleave_plan  # noqa: E402


def _runs(rng, n, choices, lo, hi):
    out, cur = [], rng.choice(choices)
    while len(out) < n:
        out += [cur] * rng.randint(lo, hi)
        cur = rng.choice([c for c in choices if c != cur] or choices)
    return out[:n]


def layouts(seed):
    rng, plans = random.Random(seed), []
    for _ in range(5):
        plan = tiny_gpt_plan(**PP.KW, num_gpus=(2,), tp=[2])
        n = plan["num_ops_in_each_stage"][0]
        tp = _runs(rng, n, [1, 2], 1, 9)
        rc = _runs(rng, n, [0, 1], 1, 7)
        plan.update(model_parallel_size_of_each_op=[tp], data_parallel_size_of_each_op=[[2 // t for t in tp]],
                    algo_of_each_op=[[rng.randint(0, 1) for _ in range(n)]], resharding_stages=[True],
                    recompute_ops=[rc])
        plans.append(plan)
    run_ranks(PP._fuzz_worker, 2, plans, PP._base(), timeout=400)


def cuts(seed):
    rng, plans = random.Random(seed), []
    kw = dict(layers=2, seq=64, hidden=64, heads=4, head_dim=16, vocab=256, global_bs=8, micro_bs=4)
    n = len(tiny_gpt_plan(**kw)["algo_of_each_op"][0])
    for _ in range(5):
        num_gpus = rng.choice([(2, 2), (1, 1, 2), (2, 1, 1), (1, 2, 1), (1, 1, 1, 1)])
        c = sorted(rng.sample(range(1, n), len(num_gpus) - 1))
        counts = [b - a for a, b in zip([0] + c, c + [n])]
        tp = [rng.choice([t for t in (1, 2) if t <= g]) for g in num_gpus]
        plans.append(tiny_gpt_plan(**kw, num_gpus=num_gpus, tp=tp, ops_per_stage=counts, recompute=rng.randint(0, 1)))
    run_ranks(PP._fuzz4_worker, 4, plans, PP._fuzz4_losses(tiny_gpt_plan(**kw)), timeout=400)


def interleaved(seed):
    rng, plans = random.Random(seed), []
    for gpus, tp in (((2, 2), [2, 2]), ((2, 2), [1, 2]), ((2, 2), [1, 1])):
        v = rng.choice([2, 3])
        base = tiny_gpt_plan(**IL.KW, num_gpus=gpus, tp=tp, recompute=rng.randint(0, 1))
        n = sum(base["num_ops_in_each_stage"])
        c = sorted(rng.sample(range(1, n), len(gpus) * v - 1))
        plans.append(interleave_plan(base, v, [b - a for a, b in zip([0] + c, c + [n])]))
    run_ranks(IL._fuzz_worker, 4, plans, IL._losses(tiny_gpt_plan(**IL.KW)), timeout=400)


def t5(seed):
    rng, plans = random.Random(seed), []
    n = len(tiny_t5_plan(layers=2)["algo_of_each_op"][0])
    for _ in range(4):
        num_gpus = rng.choice([(1, 1, 1, 1), (2, 1, 1), (1, 1, 2), (1, 2, 1), (2, 2)])
        c = sorted(rng.sample(range(1, n), len(num_gpus) - 1))
        counts = [b - a for a, b in zip([0] + c, c + [n])]
        tp = [rng.choice([t for t in (1, 2) if t <= g]) for g in num_gpus]
        plans.append(tiny_t5_plan(layers=2, num_gpus=num_gpus, tp=tp, ops_per_stage=counts, recompute=rng.randint(0, 1)))
    run_ranks(PP._t5_fuzz_worker, 4, plans, PP._other_model_losses("t5", tiny_t5_plan(layers=2), steps=2), timeout=400)


def bert(seed):
    """BERT on a padded batch: layouts, algorithms and recompute flags change inside the stage (so attention runs
    both as one kernel and as four separate ops, on all or on half of the samples), or the ops are cut into stages."""
    import test_bert_cpu as BT
    from helpers import tiny_bert_plan
    rng, plans = random.Random(seed), {}
    n = len(tiny_bert_plan(**BT.KW)["algo_of_each_op"][0])
    for k in range(3):
        plan = tiny_bert_plan(**BT.KW, num_gpus=(2,), tp=[2])
        tp = _runs(rng, n, [1, 2], 1, 9)
        tp[-1] = 2      # the head sees the whole micro-batch: a data-parallel head averages per-rank means over the
        # masked positions, which is a (slightly) different loss when the ranks hold different numbers of them
        plan.update(model_parallel_size_of_each_op=[tp], data_parallel_size_of_each_op=[[2 // t for t in tp]],
                    algo_of_each_op=[[rng.randint(0, 1) for _ in range(n)]], resharding_stages=[True],
                    recompute_ops=[[0] + _runs(rng, n - 3, [0, 1], 1, 7) + [0, 0]])
        plans[f"layouts{k}"] = plan
    c = rng.randint(1, n - 1)
    plans["cut"] = tiny_bert_plan(**BT.KW, num_gpus=(1, 1), ops_per_stage=[c, n - c], recompute=rng.randint(0, 1))
    run_ranks(BT._worker, 2, plans, BT._losses(tiny_bert_plan(**BT.KW)), timeout=600)


KINDS = {"layouts": layouts, "cuts": cuts, "interleaved": interleaved, "t5": t5, "bert": bert}

if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--first-seed", type=int, default=0)
    ap.add_argument("--seeds", type=int, default=5)
    ap.add_argument("--kinds", nargs="+", default=list(KINDS), choices=list(KINDS))
    a = ap.parse_args()
    failed = 0
    for seed in range(a.first_seed, a.first_seed + a.seeds):
        for kind in a.kinds:
            try:
                KINDS[kind](seed)
                print(kind, seed, "ok", flush=True)
            except AssertionError as e:
                failed += 1
                print(kind, seed, "FAIL", str(e)[-800:], flush=True)
    sys.exit(1 if failed else 0)
