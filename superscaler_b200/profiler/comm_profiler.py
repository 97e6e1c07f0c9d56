"""Collective profiler: times all-gather / all-reduce / reduce-scatter / all-to-all on every group size and on
every message size the cost model will look up, and writes ``prim_{model}_{size}_{collective}_{n}gpus.csv``
(``data_size(MB),time(ms)``), the format of the reference (profiler/comm_profiler.py:160-169).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m superscaler_b200.profiler.comm_profiler --model-name gpt --model-size 1_3B --prof-path <db>/

Message sizes are the distinct (rounded, MB) input sizes found in the op tables of the database, as in the
reference (profiler/comm_profiler.py:197-210): the cost model looks collectives up by exact integer MB.
Every group of n = 2, 4, ... ranks (the first n ranks of the job) is measured with CUDA events, max over ranks.
With `--impl fused` the in-kernel peer-memory collectives of this framework are timed instead of NCCL.
"""
from __future__ import annotations

import argparse
import csv
import glob
import statistics

import torch
import torch.distributed as dist

from ..parallel.state import init_distributed

PRIMS = {"gpt": ["all_gather", "all_reduce", "reduce_scatter", "all_to_all"], "resnet": ["all_gather", "all_to_all"],
         "bert": ["all_gather", "all_reduce", "reduce_scatter", "all_to_all"],
         "vit": ["all_gather", "all_reduce", "reduce_scatter", "all_to_all"], "t5": []}


def sizes_from_db(path: str, model: str, size: str, max_mb: float):
    found = set()
    for f in glob.glob(f"{path}{model}_{size}_mbs*_tp*_algo*.csv"):
        with open(f) as fh:
            for row in list(csv.reader(fh))[1:]:
                for col in (3, 6):
                    try:
                        v = float(row[col])
                    except (ValueError, IndexError):
                        continue
                    if 0 < v <= max_mb:
                        found.add(int(float("{:.0f}".format(v))))
    found.discard(0)
    return sorted(found)


def run_collective(prim: str, numel: int, group, n: int, dtype, device):
    x = torch.randn(numel, device=device).to(dtype)
    if prim == "all_reduce":
        return lambda: dist.all_reduce(x, group=group)
    if prim == "all_gather":
        out = torch.empty(numel * n, dtype=dtype, device=device)
        return lambda: dist.all_gather_into_tensor(out, x, group=group)
    if prim == "reduce_scatter":
        out = torch.empty(max(numel // n, 1), dtype=dtype, device=device)
        xin = x[: out.numel() * n]
        return lambda: dist.reduce_scatter_tensor(out, xin, group=group)
    if prim == "all_to_all":
        out = torch.empty_like(x)
        return lambda: dist.all_to_all_single(out, x[: (numel // n) * n], group=group) if numel % n == 0 else None
    raise ValueError(prim)


def time_ms(fn, warmup=5, repeat=20) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(repeat):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--model-size", required=True)
    ap.add_argument("--prof-path", required=True)
    ap.add_argument("--max-data-size", type=float, default=4096, help="MB; larger messages get the 1e9 sentinel")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    args = ap.parse_args(argv)
    rank, world, local = init_distributed()
    device = torch.device("cuda", local)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    esize = 2 if dtype == torch.bfloat16 else 4
    sizes = sizes_from_db(args.prof_path, args.model_name, args.model_size, 1e12)
    n = 2
    while n <= world:
        group = dist.new_group(list(range(n)))
        for prim in PRIMS[args.model_name]:
            rows = [["data_size(MB)", "time(ms)"]]
            for mb in sizes:
                if mb > args.max_data_size:
                    rows.append([mb, 1e9])
                    continue
                t = torch.zeros(1, device=device)
                if rank < n:
                    numel = int(mb * 1024 * 1024 / esize) // n * n
                    t[0] = time_ms(run_collective(prim, numel, group, n, dtype, device))
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                rows.append([mb, f"{t.item():.4f}"])
            if rank == 0:
                with open(f"{args.prof_path}prim_{args.model_name}_{args.model_size}_{prim}_{n}gpus.csv", "w",
                          newline="") as f:
                    csv.writer(f).writerows(rows)
        n *= 2
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
