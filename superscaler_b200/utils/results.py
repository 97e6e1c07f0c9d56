"""Result collection: throughput from the runtime CSVs, search cost from the search summaries, and cost-model
accuracy (predicted vs measured iteration time / memory).

Counterparts of scripts/get_e2e_performance.py, get_search_cost.py, get_perf_model_acc.py and get_common.py of
the reference.  One deliberate difference: an iteration ends when its SLOWEST rank ends, so the iteration time
of a run is the maximum over the rank CSVs (the reference reports the fastest rank, scripts/get_common.py:36-55).
"""
from __future__ import annotations

import csv
import glob
import os
from typing import Dict, Optional, Tuple


def read_runtime_csv(path: str) -> Dict[str, float]:
    with open(path) as f:
        rows = list(csv.reader(f))
    return {k: float(v) for k, v in zip(rows[0], rows[1])}


def run_iteration_time_ms(log_path: str, config_name: str) -> Optional[float]:
    files = glob.glob(os.path.join(log_path, "csv", f"{config_name}_stage*_rank*.csv"))
    if not files:
        return None
    return max(read_runtime_csv(f)["time"] for f in files)


def throughput(log_path: str, config_name: str) -> Optional[float]:
    """samples / s = global batch size / iteration time."""
    files = glob.glob(os.path.join(log_path, "csv", f"{config_name}_stage*_rank*.csv"))
    if not files:
        return None
    gbs = read_runtime_csv(files[0])["global_batch_size"]
    return gbs / (run_iteration_time_ms(log_path, config_name) / 1000.0)


def best_throughput(log_path: str) -> Tuple[Optional[str], float]:
    names = {os.path.basename(f).rsplit("_stage", 1)[0] for f in glob.glob(os.path.join(log_path, "csv", "*_stage*_rank*.csv"))}
    best, best_t = None, 0.0
    for n in sorted(names):
        t = throughput(log_path, n) or 0.0
        if t > best_t:
            best, best_t = n, t
    return best, best_t


def throughput_table(log_path: str) -> str:
    """Markdown table of every run under log_path/csv: iteration time (slowest rank), samples / s, peak memory over
    the stages (the text counterpart of the reference's result CSVs and plots, scripts/get_e2e_performance.py and
    scripts/plot_fig*.py; no plotting library is assumed here)."""
    names = sorted({os.path.basename(f).rsplit("_stage", 1)[0]
                    for f in glob.glob(os.path.join(log_path, "csv", "*_stage*_rank*.csv"))})
    lines = ["| run | ranks | iteration (ms) | samples / s | peak memory (MB) |", "|---|---|---|---|---|"]
    for n in names:
        ranks = len(glob.glob(os.path.join(log_path, "csv", f"{n}_stage*_rank*.csv")))
        mem = stage_memory_mb(log_path, n)
        lines.append(f"| {n} | {ranks} | {run_iteration_time_ms(log_path, n):.1f} | {throughput(log_path, n):.2f} | "
                     f"{max(mem.values()) if mem else 0:.0f} |")
    return "\n".join(lines)


def search_cost(log_path: str, model: str, size: str) -> Optional[float]:
    files = sorted(glob.glob(os.path.join(log_path, f"{model}_{size}_summary_*.csv")))
    if not files:
        return None
    with open(files[-1]) as f:
        rows = list(csv.reader(f))
    return float(rows[1][0])


def stage_memory_mb(log_path: str, config_name: str) -> Dict[int, float]:
    out: Dict[int, float] = {}
    for f in glob.glob(os.path.join(log_path, "csv", f"{config_name}_stage*_rank*.csv")):
        stage = int(os.path.basename(f).rsplit("_stage", 1)[1].split("_rank")[0])
        out[stage] = max(out.get(stage, 0.0), read_runtime_csv(f)["max_allocated_memory(MB)"])
    return out


def cost_model_accuracy(pred_csv: str, log_path: str, config_name: str) -> Dict[str, float]:
    """Compares the search's per-stage prediction (info_*.csv) with a run: max stage time and max memory."""
    with open(pred_csv) as f:
        rows = list(csv.reader(f))[1:]
    pred_time = max(float(r[1]) for r in rows)
    pred_mem = max(float(r[2]) for r in rows)
    actual = run_iteration_time_ms(log_path, config_name)
    mem = stage_memory_mb(log_path, config_name)
    out = {"predicted_time_ms": pred_time, "predicted_memory_mb": pred_mem}
    if actual is not None:
        out["actual_time_ms"] = actual
        out["time_error_pct"] = abs(pred_time - actual) / actual * 100.0
    if mem:
        out["actual_memory_mb"] = max(mem.values())
    return out


def main(argv=None) -> None:
    """`python -m superscaler_b200.utils.results --log-path logs/ [--config NAME] [--pred-csv info.csv]`:
    throughput of every run under logs/csv (or of one), and the cost-model error when a prediction CSV is given."""
    import argparse
    import json
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--log-path", required=True)
    ap.add_argument("--config", default=None)
    ap.add_argument("--pred-csv", default=None)
    ap.add_argument("--table", action="store_true", help="markdown table of all runs under the log path")
    a = ap.parse_args(argv)
    if a.table:
        print(throughput_table(a.log_path))
        return
    if a.config is None:
        name, t = best_throughput(a.log_path)
        print(json.dumps({"best_config": name, "samples_per_s": t}))
        return
    out = {"config": a.config, "samples_per_s": throughput(a.log_path, a.config),
           "iteration_ms": run_iteration_time_ms(a.log_path, a.config), "memory_mb": stage_memory_mb(a.log_path, a.config)}
    if a.pred_csv:
        out["cost_model"] = cost_model_accuracy(a.pred_csv, a.log_path, a.config)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
