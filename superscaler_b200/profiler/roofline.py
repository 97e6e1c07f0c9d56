"""Roofline report of a profiled GPT op table: for every fused op group of one transformer layer (and the
embedding / LM head), the algorithmic FLOPs or bytes of the group, the time the database records, and the
achieved rate as a fraction of a measured peak.

    python -m superscaler_b200.profiler.roofline --profiled-time-path profiled-time-b200/ --model-size 1_3B \
        --mbs 16 [--tp 1] [--peak-tflops 1384.9] [--peak-gbs 6555.5]

GEMM-shaped groups are set against the matrix-multiply peak (pass the SUSTAINED figure: the tables are measured
with calls launched back to back under the power cap), the others against the copy bandwidth.  FLOPs count a
multiply-add as 2; the backward of a linear layer is two GEMMs (input and weight gradient), the backward of
attention 2.5 times its forward; causal attention counts half of the score matrix.
"""
from __future__ import annotations

import argparse
import csv
from typing import Dict, List, Tuple

from ..search import config as sc


def _table(path: str) -> Dict[str, Tuple[float, float]]:
    with open(path) as f:
        rows = list(csv.reader(f))[1:]
    return {r[0]: (float(r[1]), float(r[2])) for r in rows}


def gpt_groups(size: str, mbs: int, tp: int, b200_shapes: bool = True) -> List[tuple]:
    """(table row, description, kind, forward work, backward work): work in FLOPs for kind 'gemm', bytes for 'mem'."""
    table = sc.B200_GPT_SIZES if (b200_shapes and size in sc.B200_GPT_SIZES) else sc.GPT_SIZES
    _, s, h, ffn, heads, hd, vocab, _ = table[size]
    T = mbs * s
    act = T * h * 2                      # one bf16 activation matrix, bytes
    qkv = 2 * T * h * (3 * heads * hd) / tp
    attn = 4 * mbs * (heads / tp) * s * s * hd * 0.5
    dense = 2 * T * (heads * hd) * h / tp
    mlp = 2 * (2 * T * h * ffn) / tp
    head = 2 * T * h * vocab / tp
    return [
        ("encoder-embedding", "embedding (word + position + dropout)", "mem", 2 * act, 2 * act),
        ("enc-1st-layernorm", "LayerNorm", "mem", 2 * act, 3 * act),
        ("enc-attention-qkv", "QKV GEMM + bias", "gemm", qkv, 2 * qkv),
        ("enc-attention-score", "flash attention (score, softmax, dropout, context)", "gemm", attn, 2.5 * attn),
        ("enc-attention-dense", "output GEMM + bias + dropout + residual", "gemm", dense, 2 * dense),
        ("enc-2nd-layernorm", "LayerNorm", "mem", 2 * act, 3 * act),
        ("enc-MLP-GEMM-1", "MLP: GEMM + bias + GeLU, GEMM + bias + dropout + residual", "gemm", mlp, 2 * mlp),
        ("gpt-post-process", "LM head GEMM + cross entropy", "gemm", head, 2 * head),
    ]


def report(db: str, size: str, mbs: int, tp: int, peak_tflops: float, peak_gbs: float, algo: int = 0) -> str:
    rows = _table(f"{db}gpt_{size}_mbs{mbs}_tp{tp}_algo{algo}.csv")
    out = [f"| op group (table row) | forward | of peak | backward | of peak |", "|---|---|---|---|---|"]
    layer_us = [0.0, 0.0]
    for name, what, kind, wf, wb in gpt_groups(size, mbs, tp):
        tf, tb = rows[name]
        cells = []
        for t_us, work in ((tf, wf), (tb, wb)):
            if kind == "gemm":
                rate = work / (t_us * 1e-6) / 1e12
                cells += [f"{t_us:.0f} us, {rate:.0f} TFLOP/s", f"{rate / peak_tflops:.2f}"]
            else:
                rate = work / (t_us * 1e-6) / 1e9
                cells += [f"{t_us:.0f} us, {rate:.0f} GB/s", f"{rate / peak_gbs:.2f}"]
        if name.startswith("enc-"):
            layer_us[0] += tf
            layer_us[1] += tb
        out.append(f"| {what} (`{name}`) | {cells[0]} | {cells[1]} | {cells[2]} | {cells[3]} |")
    out.append("")
    out.append(f"One transformer layer: {layer_us[0]:.0f} us forward + {layer_us[1]:.0f} us backward.")
    return "\n".join(out)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--profiled-time-path", required=True)
    ap.add_argument("--model-size", default="1_3B")
    ap.add_argument("--mbs", type=int, default=16)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--peak-tflops", type=float, default=1384.9, help="measured sustained bf16 matrix-multiply rate")
    ap.add_argument("--peak-gbs", type=float, default=6555.5, help="measured copy bandwidth")
    a = ap.parse_args(argv)
    print(report(a.profiled_time_path, a.model_size, a.mbs, a.tp, a.peak_tflops, a.peak_gbs))


if __name__ == "__main__":
    main()
