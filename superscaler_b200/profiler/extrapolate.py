"""Op tables for a GPT size that has not been profiled, scaled from the tables of one that has.

    python -m superscaler_b200.profiler.extrapolate --from-path profiled-time-b200/ --to-path <out>/ \
        --from-size 1_3B --to-size 13B

All GPT sizes share the sequence length, the vocabulary and the ratios ffn = 4 h and heads x head_dim = h, so with
r = h_to / h_from every entry of a table scales by a power of r that its meaning fixes:

  * time of the linear layers (QKV, attention output, MLP)      r^2   (FLOPs ~ tokens x h^2)
  * time of attention, LayerNorm, embedding, LM head + loss      r     (FLOPs or bytes ~ tokens x h)
  * input / output / activation / workspace sizes                r
  * weights of the linear layers                                 r^2, of embedding, LayerNorm and LM head: r

i.e. the measured kernels are assumed to keep their efficiency on the larger matrices (they lose none: the GEMM
tiles only get more work per launch).  Under tensor parallelism the measured op times contain the op's collective,
whose bytes grow like r, not r^2, so scaled tensor-parallel tables are pessimistic for the linear layers.  The
collective tables (`prim_*`) are re-keyed for the tensor sizes of the new tables by log-log interpolation of the
measured points, the p2p table is copied.  The output directory gets an EXTRAPOLATED.md that says so: plans searched
against these tables are estimates until the size is profiled (`profiler.op_profiler`).
"""
from __future__ import annotations

import argparse
import csv
import glob
import math
import os
import shutil
from typing import List, Tuple

from ..search import config as sc

# exponent of r for (time, weights) per table row; sizes always scale with exponent 1
_QUADRATIC = ("enc-attention-qkv", "enc-attention-dense", "enc-MLP-GEMM-1", "enc-MLP-GEMM-2")


def _exponents(op: str) -> Tuple[int, int]:
    return (2, 2) if op in _QUADRATIC else (1, 1)


def scale_table(rows: List[List[str]], r: float) -> List[List[str]]:
    """rows: a table without its header; columns op, fwd us, bwd us, in, out, weights, activations, reserved fwd,
    reserved bwd[, overlapped fwd comm, overlapped bwd comm]."""
    out = []
    for row in rows:
        t_exp, w_exp = _exponents(row[0])
        vals = [float(x) for x in row[1:]]
        scaled = [vals[0] * r ** t_exp, vals[1] * r ** t_exp, vals[2] * r, vals[3] * r, vals[4] * r ** w_exp,
                  vals[5] * r, vals[6] * r, vals[7] * r]
        scaled += [v * r for v in vals[8:]]
        out.append([row[0]] + [f"{v:.3f}" for v in scaled])
    return out


def _interpolate(points: List[Tuple[float, float]], size: float) -> float:
    """Time (ms) of a collective of `size` MB from measured (size, time) points: log-log linear between neighbours,
    the end segments extended outwards."""
    pts = sorted(p for p in points if p[0] > 0 and p[1] > 0)
    if not pts:
        return 0.0
    if len(pts) == 1:
        return pts[0][1] * size / pts[0][0]
    lo, hi = pts[0], pts[1]
    for a, b in zip(pts, pts[1:]):
        lo, hi = a, b
        if size <= b[0]:
            break
    slope = math.log(hi[1] / lo[1]) / math.log(hi[0] / lo[0])
    return lo[1] * (size / lo[0]) ** slope


def extrapolate(from_path: str, to_path: str, from_size: str, to_size: str) -> List[str]:
    h_from, h_to = sc.GPT_SIZES[from_size][2], sc.GPT_SIZES[to_size][2]
    if from_size in sc.B200_GPT_SIZES:
        h_from = sc.B200_GPT_SIZES[from_size][2]
    r = h_to / h_from
    os.makedirs(to_path, exist_ok=True)
    written, sizes_mb = [], set()
    for src in sorted(glob.glob(os.path.join(from_path, f"gpt_{from_size}_mbs*_tp*_algo*.csv"))):
        with open(src) as f:
            rows = list(csv.reader(f))
        heads = sc.GPT_SIZES[to_size][4]
        tp = int(os.path.basename(src).split("_tp")[1].split("_")[0])
        if heads % tp:
            continue        # the head count of the target does not divide over this group
        scaled = scale_table(rows[1:], r)
        dst = os.path.join(to_path, os.path.basename(src).replace(f"gpt_{from_size}_", f"gpt_{to_size}_"))
        with open(dst, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(rows[0])
            w.writerows(scaled)
        written.append(dst)
        for row in scaled:
            for v in (row[3], row[4], row[6]):     # the cost model looks a size up rounded to whole MB
                sizes_mb.update((int(float(v)), int(round(float(v)))))
    for src in sorted(glob.glob(os.path.join(from_path, f"prim_gpt_{from_size}_*gpus.csv"))):
        with open(src) as f:
            rows = list(csv.reader(f))
        points = [(float(a), float(b)) for a, b in rows[1:] if float(b) < 1e8]
        dst = os.path.join(to_path, os.path.basename(src).replace(f"gpt_{from_size}_", f"gpt_{to_size}_"))
        with open(dst, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(rows[0])
            for s in sorted(x for x in sizes_mb if x > 0):
                w.writerow([s, f"{_interpolate(points, s):.4f}"])
        written.append(dst)
    for name in ("p2p_intra_node.csv", "p2p_inter_node.csv"):
        if os.path.exists(os.path.join(from_path, name)):
            shutil.copy(os.path.join(from_path, name), os.path.join(to_path, name))
    with open(os.path.join(to_path, "EXTRAPOLATED.md"), "a") as f:
        f.write(f"gpt_{to_size}: scaled from the measured gpt_{from_size} tables of {from_path} by "
                f"`python -m superscaler_b200.profiler.extrapolate` (hidden size ratio {r:.3f}); estimates, not "
                f"measurements.\n")
    return written


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--from-path", required=True)
    ap.add_argument("--to-path", required=True)
    ap.add_argument("--from-size", default="1_3B")
    ap.add_argument("--to-size", required=True)
    a = ap.parse_args(argv)
    files = extrapolate(a.from_path, a.to_path, a.from_size, a.to_size)
    print(f"wrote {len(files)} tables for gpt_{a.to_size} under {a.to_path}")


if __name__ == "__main__":
    main()
