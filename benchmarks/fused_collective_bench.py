"""Fused compute + collective micro-benchmark (the resharding / fused-collective configuration of the benchmark
suite), stand-alone:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        benchmarks/fused_collective_bench.py [--mbs 1 4 8] [--hidden 2048 4096 8192] [--iters 20]

Runs superscaler_b200.profiler.fused_bench at tensor-parallel degree N: a self-check of the three fused kernels
against GEMM + NCCL, then per shape one JSON line for GEMM -> all-reduce, GEMM -> reduce-scatter and all-gather -> GEMM
(fused time, NCCL-path time, NVLink bytes per GPU, achieved GB/s, roofline fraction).  `bench.py` runs the same
block, on two shapes, before its timed regions whenever it is started on 2 or more GPUs.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mbs", type=int, nargs="+", default=[1, 4, 8])
    ap.add_argument("--hidden", type=int, nargs="+", default=[2048, 4096, 8192])
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    from superscaler_b200.parallel.state import init_distributed
    from superscaler_b200.parallel.symm import FusedTPContext
    from superscaler_b200.profiler import fused_bench
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    ctx = FusedTPContext(None, max(a.mbs) * a.seq, max(a.hidden), dev)
    check = fused_bench.self_check(ctx, dev, rank, world)
    if rank == 0:
        print(json.dumps({"self_check": check}), flush=True)
    for row in fused_bench.microbench(ctx, dev, rank, world, mbs_list=a.mbs, hidden_list=a.hidden, seq=a.seq,
                                      warmup=a.warmup, iters=a.iters):
        if rank == 0:
            print(json.dumps(row), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
