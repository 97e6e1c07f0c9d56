"""Stand-alone predictor: time / memory breakdown of one plan JSON under a profiled database.

    python -m superscaler_b200.search.predict --initial-point plan.json --profiled-time-path <db>/ \
        --num-nodes 1 --num-gpus-per-node 8 [--save-to-csv out.csv]

(reference: `python3 aceso_cost_model.py --initial-point cfg.json`, search/aceso_cost_model.py:926-932).
"""
from __future__ import annotations

import argparse

from .config import load_plan, write_stage_info_csv
from .context import SearchContext, add_cli_arguments, args_from_namespace


def predict(args):
    ctx = SearchContext(args)
    plan, _ = load_plan(args.initial_point, ctx.full_op_list)
    report: list = []
    ctx.cost.evaluate(plan, report)
    return ctx, plan, report


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_cli_arguments(p)
    args = args_from_namespace(p.parse_args(argv))
    ctx, plan, report = predict(args)
    print("overall time = {:.2f} ms".format(max(plan.time_list)))
    print("stage, fwd, bwd+recompute, recompute, in_comm(+reshard), out_comm(+reshard), reshard, pipeline time (ms)")
    worst = max(range(plan.num_stages), key=lambda i: plan.time_list[i])
    for r in report:
        mark = " * " if r["stage"] == worst else ""
        print(f"{mark}[stage {r['stage']}], {r['fwd_ms']:.2f}, {r['bwd_ms']:.2f}, {r['recompute_ms']:.2f}, "
              f"{r['in_comm_ms']:.2f}, {r['out_comm_ms']:.2f}, {r['reshard_ms']:.2f}, {r['pipeline_time_ms']:.2f}")
    print("\nmax allocated memory = {:.2f} MB".format(max(plan.memory_list)))
    for r in report:
        print(f"[stage {r['stage']}] memory = {r['memory_mb']:.2f} MB. weights = {r['weights_mb']:.0f}, gradients = "
              f"{r['grads_mb']:.0f}, optimizer = {r['optimizer_mb']:.0f}, activations = {r['activations_mb']:.0f}, "
              f"peak += {r['peak_mb']:.0f}, memory_reserved = {r['reserved_mb']:.0f}")
    if args.save_to_csv is not None:
        write_stage_info_csv(plan, ctx.cost.reserved_list(plan), args.save_to_csv)


if __name__ == "__main__":
    main()
