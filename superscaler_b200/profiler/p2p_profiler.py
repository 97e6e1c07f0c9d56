"""Point-to-point bandwidth profiler: rank 0 sends 1 MB ... 1 GB messages to rank 1 and the measured bandwidth
(GB/s) is written as the two-row CSV the cost model reads (sizes; bandwidths) -- ``p2p_intra_node.csv`` or
``p2p_inter_node.csv`` (reference: profiler/p2p_band_profiler.py:14-62).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m superscaler_b200.profiler.p2p_profiler --prof-path <db>/ [--inter-node]
"""
from __future__ import annotations

import argparse
import csv

import torch
import torch.distributed as dist

from ..parallel.state import init_distributed


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--prof-path", required=True)
    ap.add_argument("--inter-node", action="store_true")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--repeat", type=int, default=50)
    args = ap.parse_args(argv)
    rank, world, local = init_distributed()
    assert world >= 2
    device = torch.device("cuda", local)
    sizes = [2 ** i for i in range(11)]  # MB
    bands = []
    for mb in sizes:
        x = torch.empty(mb * 1024 * 1024 // 2, dtype=torch.bfloat16, device=device)

        def once():
            if rank == 0:
                dist.send(x, 1)
            elif rank == 1:
                dist.recv(x, 0)

        for _ in range(args.warmup):
            once()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.repeat):
            once()
        e1.record()
        e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.repeat], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        bands.append(mb / 1024.0 / (t.item() / 1000.0))
    if rank == 0:
        name = "p2p_inter_node.csv" if args.inter_node else "p2p_intra_node.csv"
        with open(args.prof_path + name, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(sizes)
            w.writerow([f"{b:.3f}" for b in bands])
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
