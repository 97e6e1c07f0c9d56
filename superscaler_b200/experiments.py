"""Experiment driver: the search / execute / collect / plot workflow of the evaluation, for the three models and
the three experiment sizes, as one command-line tool over this package's own entry points.

    python -m superscaler_b200.experiments search   --model gpt --mode small
    python -m superscaler_b200.experiments baseline --model gpt --mode small        # uniform grid planner
    python -m superscaler_b200.experiments execute  --model gpt --mode small [--system aceso|grid]
    python -m superscaler_b200.experiments collect  --mode small                    # tables + CSV files
    python -m superscaler_b200.experiments plot     --mode small                    # SVG figures from the CSV files
    python -m superscaler_b200.experiments all      --mode small                    # everything above, all models

Counterparts in the reference: scripts/aceso_{gpt,t5,resnet}_{search,execute}.sh with their `small`, `large` and
`scale` settings (scripts/aceso_gpt_search.sh:5-184), scripts/megatron_*_{search,execute}.sh for the grid-planned
baseline, scripts/run_all_small.sh, scripts/get_{e2e_performance,search_cost,perf_model_acc}.py and
scripts/plot_fig{7,8,9,15,16}*.py.  Differences: one Python tool instead of 30 shell scripts; runs are launched
with torch.distributed.run on this node (the multi-node `large` cases are capped at the GPUs of one node unless
--num-nodes is given); figures are written as SVG by a few lines of plain Python (no plotting library is assumed).

Settings (per model: size, nodes, GPUs per node):
  small : GPT 1.3B / T5 770M / Wide-ResNet 1B on 1 x 4 GPUs, global batch 512 / 512 / 768, memory limit 12000 MB
          against the 4-GPU database (the reference's profiled-time-miniset), or `--shapes b200` against
          profiled-time-b200 with the B200 memory limit
  large : GPT 350M..13B, T5 770M..22B, Wide-ResNet 500M..13B on 1, 4, 8, 16, 32 GPUs, global batch 1024 / 1024 /
          1536, memory limit 28000 MB (the 1-GPU point is searched like the others: one stage, one GPU)
  scale : GPT with 8..1024 layers on 8 GPUs ("scale-layer"), global batch 1024
"""
from __future__ import annotations

import argparse
import csv
import glob
import os
import subprocess
import sys
import time
from typing import Dict, List, Optional, Tuple

from .utils import results

GLOBAL_BATCH = {"small": {"gpt": 512, "t5": 512, "resnet": 768}, "large": {"gpt": 1024, "t5": 1024, "resnet": 1536},
                "scale": {"gpt": 1024}}
MICRO_BATCHES = {"gpt": [1, 2, 4, 8], "t5": [1, 2, 4, 8], "resnet": [16, 32, 48, 64]}
MEMORY_LIMIT = {"small": 12000, "large": 28000, "scale": 28000}
B200_MEMORY_LIMIT = 170000
# (model size, nodes, GPUs per node)
CASES = {
    "small": {"gpt": [("1_3B", 1, 4)], "t5": [("770M", 1, 4)], "resnet": [("1B", 1, 4)]},
    "large": {"gpt": [("350M", 1, 1), ("1_3B", 1, 4), ("2_6B", 1, 8), ("6_7B", 2, 8), ("13B", 4, 8)],
              "t5": [("770M", 1, 1), ("3B", 1, 4), ("6B", 1, 8), ("11B", 2, 8), ("22B", 4, 8)],
              "resnet": [("500M", 1, 1), ("2B", 1, 4), ("4B", 1, 8), ("6_8B", 2, 8), ("13B", 4, 8)]},
    "scale": {"gpt": [(f"{n}layers", 1, 8) for n in (8, 16, 32, 64, 128, 256, 512, 1024)]},
}


def _dirs(root: str, system: str, model: str, size: str) -> Tuple[str, str, str]:
    base = os.path.join(root, system)
    log = os.path.join(base, "search", model, size) + "/"
    cfg = os.path.join(base, "configs", model, size) + "/"
    run = os.path.join(base, "runtime", model, size) + "/"
    for d in (log + "trends", cfg + "top_configs", cfg + "csv", run + "csv"):
        os.makedirs(d, exist_ok=True)
    return log, cfg, run


def _run(cmd: List[str], dry: bool) -> int:
    print("+ " + " ".join(cmd), flush=True)
    if dry:
        return 0
    return subprocess.call(cmd)


def cases(mode: str, model: str, max_gpus: Optional[int]) -> List[Tuple[str, int, int]]:
    out = []
    for size, nodes, gpn in CASES[mode].get(model, []):
        if max_gpus is not None and nodes * gpn > max_gpus:
            continue
        out.append((size, nodes, gpn))
    return out


def search(a, system: str = "aceso") -> None:
    """One search (or grid plan) per case of the mode."""
    for size, nodes, gpn in cases(a.mode, a.model, a.max_gpus):
        log, cfg, _ = _dirs(a.results, system, a.model, size)
        layers = []
        model_size = size
        if a.mode == "scale":
            layers = ["--num-layers", size.replace("layers", "")]
            model_size = "1_3B"                      # width of the scaled model; its depth comes from --num-layers
        module = "superscaler_b200.search.search" if system == "aceso" else "superscaler_b200.search.grid_plan"
        limit = B200_MEMORY_LIMIT if a.shapes == "b200" else MEMORY_LIMIT[a.mode]
        cmd = [sys.executable, "-m", module, "--model-name", a.model, "--model-size", model_size,
               "--global-batch-size", str(GLOBAL_BATCH[a.mode][a.model]), "--micro-batch-size",
               *map(str, MICRO_BATCHES[a.model]), "--num-nodes", str(nodes), "--num-gpus-per-node", str(gpn),
               "--memory-limit", str(limit), "--log-path", log, "--profiled-time-path", a.database,
               "--config-save-path", cfg, "--config-suffix", time.strftime("%Y-%m-%d-%H-%M-%S"), "--shapes", a.shapes,
               "--max-num-hops", "7", "--time-budget-total", str(a.budget), "--num-of-saved-configs", "3", *layers]
        if system == "aceso":
            cmd += ["--initial-point", a.initial_point]
            if a.model == "resnet":
                cmd += ["--finetune-after-trial", "1"]
        _run(cmd, a.dry_run)


def execute(a) -> None:
    """Three training iterations of every saved top plan; the per-rank CSV of the last one is what `collect` reads."""
    for size, nodes, gpn in cases(a.mode, a.model, a.max_gpus):
        _, cfg, run = _dirs(a.results, a.system, a.model, size)
        plans = sorted(glob.glob(cfg + "top_configs/*.json")) or sorted(glob.glob(cfg + "*.json"))
        for plan in plans[:a.top]:
            n = nodes * gpn
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                   "--master-addr", "127.0.0.1", "--master-port", str(a.master_port), "-m",
                   "superscaler_b200.runtime.pretrain", "--flexpipe-config", plan, "--train-iters", str(a.train_iters),
                   "--eval-iters", "0", "--lr-decay-iters", "320000", "--lr", "0.00015", "--lr-decay-style", "cosine",
                   "--min-lr", "1.0e-5", "--weight-decay", "1e-2", "--clip-grad", "1.0", "--lr-warmup-fraction", ".01",
                   "--log-interval", "1", "--log-path", run]
            _run(cmd, a.dry_run)


def _pred_csv(cfg: str, name: str) -> Optional[str]:
    path = os.path.join(cfg, "csv", f"info_{name}.csv")
    return path if os.path.exists(path) else None


def collect(a) -> Dict[str, List[list]]:
    """Tables in the layout of the reference's results/*.csv: throughput per system and size (and normalised to the
    grid-planned baseline), search cost, cost-model time / memory accuracy."""
    tables: Dict[str, List[list]] = {}
    out_dir = os.path.join(a.results, "tables")
    os.makedirs(out_dir, exist_ok=True)
    for model in CASES[a.mode]:
        sizes = [s for s, _, _ in cases(a.mode, model, a.max_gpus)]
        thpt = {"grid": [], "aceso": []}
        cost = {"grid": [], "aceso": []}
        t_act, t_pred, m_act, m_pred = [], [], [], []
        for size in sizes:
            best_name = None
            for system in ("grid", "aceso"):
                log, cfg, run = _dirs(a.results, system, model, size)
                name, best = results.best_throughput(run)
                thpt[system].append(round(best, 2) if name else None)
                lookup = "1_3B" if a.mode == "scale" else size
                c = results.search_cost(log, model, lookup)
                cost[system].append(round(c, 2) if c is not None else None)
                if system == "aceso":
                    best_name, best_cfg, best_run = name, cfg, run
            pred = _pred_csv(best_cfg, best_name) if best_name else None
            if pred:
                acc = results.cost_model_accuracy(pred, best_run, best_name)
                t_act.append(round(acc.get("actual_time_ms", 0.0) / 1e3, 2))
                t_pred.append(round(acc["predicted_time_ms"] / 1e3, 2))
                m_act.append(round(acc.get("actual_memory_mb", 0.0)))
                m_pred.append(round(acc["predicted_memory_mb"]))
            else:
                for lst in (t_act, t_pred, m_act, m_pred):
                    lst.append(None)
        norm = {s: [round(v / b, 2) if v and b else None for v, b in zip(thpt[s], thpt["grid"])] for s in thpt}
        tables[f"e2e_thpt_{a.mode}_{model}"] = [["system"] + sizes, ["grid"] + thpt["grid"], ["aceso"] + thpt["aceso"]]
        tables[f"e2e_norm_thpt_{a.mode}_{model}"] = [["system"] + sizes, ["grid"] + norm["grid"], ["aceso"] + norm["aceso"]]
        tables[f"search_cost_{a.mode}_{model}"] = [["system"] + sizes, ["grid"] + cost["grid"], ["aceso"] + cost["aceso"]]
        tables[f"perf_model_time_{a.mode}_{model}"] = [["kind"] + sizes, ["actual"] + t_act, ["predicted"] + t_pred]
        tables[f"perf_model_mem_{a.mode}_{model}"] = [["kind"] + sizes, ["actual"] + m_act, ["predicted"] + m_pred]
    for name, rows in tables.items():
        with open(os.path.join(out_dir, name + ".csv"), "w", newline="") as f:
            csv.writer(f).writerows([["" if v is None else v for v in r] for r in rows])
        print(f"## {name}")
        for r in rows:
            print("| " + " | ".join("-" if v is None else str(v) for v in r) + " |")
    return tables


# ---- figures (SVG, no plotting library) ---------------------------------------------------------------------------
_COLORS = ["#4878a8", "#e49444", "#6a9f58", "#d1615d", "#85b6b2"]


def svg_grouped_bars(title: str, groups: List[str], series: Dict[str, List[Optional[float]]], ylabel: str,
                     log_y: bool = False) -> str:
    """A grouped bar chart: one group per model size, one bar per system."""
    import math
    w, h, left, bottom, top = 720, 360, 70, 50, 40
    vals = [v for s in series.values() for v in s if v]
    vmax = max(vals) if vals else 1.0
    vmin = min(vals) if vals else 0.1

    def y_of(v: float) -> float:
        if log_y:
            lo, hi = math.log10(vmin / 2), math.log10(vmax * 1.5)
            return top + (h - top - bottom) * (1 - (math.log10(v) - lo) / (hi - lo))
        return top + (h - top - bottom) * (1 - v / (vmax * 1.15))

    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" font-family="sans-serif" font-size="12">',
           f'<text x="{w / 2}" y="20" text-anchor="middle" font-size="14">{title}</text>',
           f'<text x="14" y="{h / 2}" transform="rotate(-90 14 {h / 2})" text-anchor="middle">{ylabel}</text>',
           f'<line x1="{left}" y1="{h - bottom}" x2="{w - 20}" y2="{h - bottom}" stroke="black"/>',
           f'<line x1="{left}" y1="{top}" x2="{left}" y2="{h - bottom}" stroke="black"/>']
    gw = (w - left - 20) / max(len(groups), 1)
    bw = gw * 0.8 / max(len(series), 1)
    for gi, g in enumerate(groups):
        out.append(f'<text x="{left + gw * (gi + 0.5)}" y="{h - bottom + 16}" text-anchor="middle">{g}</text>')
        for si, (name, vs) in enumerate(series.items()):
            v = vs[gi] if gi < len(vs) else None
            if not v:
                continue
            x = left + gw * gi + gw * 0.1 + bw * si
            y = y_of(v)
            out.append(f'<rect x="{x:.1f}" y="{y:.1f}" width="{bw:.1f}" height="{h - bottom - y:.1f}" '
                       f'fill="{_COLORS[si % len(_COLORS)]}"/>')
            out.append(f'<text x="{x + bw / 2:.1f}" y="{y - 3:.1f}" text-anchor="middle" font-size="10">{v:g}</text>')
    for si, name in enumerate(series):
        out.append(f'<rect x="{left + 10 + 110 * si}" y="{top - 14}" width="10" height="10" fill="{_COLORS[si % len(_COLORS)]}"/>')
        out.append(f'<text x="{left + 24 + 110 * si}" y="{top - 5}">{name}</text>')
    out.append("</svg>")
    return "\n".join(out)


def plot(a) -> List[str]:
    """Figures from the CSV tables of `collect`: throughput normalised to the grid planner (the reference's figures
    7 / 8), search cost on a log axis (figure 9), cost-model time and memory accuracy (figures 15 / 16)."""
    tdir = os.path.join(a.results, "tables")
    fdir = os.path.join(a.results, "figures")
    os.makedirs(fdir, exist_ok=True)
    written = []
    for path in sorted(glob.glob(os.path.join(tdir, f"*_{a.mode}_*.csv"))):
        name = os.path.basename(path)[:-4]
        with open(path) as f:
            rows = list(csv.reader(f))
        groups = rows[0][1:]
        series = {r[0]: [float(v) if v else None for v in r[1:]] for r in rows[1:]}
        ylabel = ("samples / s" if name.startswith("e2e_thpt") else "throughput / grid planner" if "norm" in name else
                  "search time (s)" if name.startswith("search_cost") else "iteration time (s)" if "time" in name
                  else "memory (MB)")
        svg = svg_grouped_bars(name, groups, series, ylabel, log_y=name.startswith("search_cost"))
        out = os.path.join(fdir, name + ".svg")
        with open(out, "w") as f:
            f.write(svg)
        written.append(out)
    print("\n".join(written))
    return written


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=["search", "baseline", "execute", "collect", "plot", "all"])
    ap.add_argument("--model", default="gpt", choices=["gpt", "t5", "resnet"])
    ap.add_argument("--mode", default="small", choices=["small", "large", "scale"])
    ap.add_argument("--system", default="aceso", choices=["aceso", "grid"], help="whose plans `execute` runs")
    ap.add_argument("--database", default=None, help="profiled database (default: profiled-time-b200/ with --shapes b200)")
    ap.add_argument("--shapes", default="b200", choices=["b200", "reference"])
    ap.add_argument("--results", default="./logs", help="root of search logs, plans, runtime CSVs, tables and figures")
    ap.add_argument("--initial-point", default="balance",
                       help="balance (the reference's scripts), imbalance_gpu, imbalance_op, grid (start from the best "
                            "uniform plan: never slower than the baseline), both (balance and grid, the faster "
                            "result is kept) or a plan JSON")
    ap.add_argument("--budget", type=int, default=200, help="search time budget per stage count (s)")
    ap.add_argument("--max-gpus", type=int, default=None, help="skip cases that need more GPUs than this")
    ap.add_argument("--top", type=int, default=3, help="how many saved plans per case `execute` runs")
    ap.add_argument("--train-iters", type=int, default=3)
    ap.add_argument("--master-port", type=int, default=29500)
    ap.add_argument("--dry-run", action="store_true", help="print the commands without running them")
    a = ap.parse_args(argv)
    if a.database is None:
        here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        a.database = os.path.join(here, "profiled-time-b200") + "/"
    if a.command == "search":
        search(a, "aceso")
    elif a.command == "baseline":
        search(a, "grid")
    elif a.command == "execute":
        execute(a)
    elif a.command == "collect":
        collect(a)
    elif a.command == "plot":
        plot(a)
    else:
        for model in CASES[a.mode]:
            a.model = model
            search(a, "aceso")
            search(a, "grid")
            for system in ("aceso", "grid"):
                a.system = system
                execute(a)
        collect(a)
        plot(a)


if __name__ == "__main__":
    main()
