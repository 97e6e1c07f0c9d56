"""Resharding micro-benchmark: one activation walks down the layouts tp N -> N/2 -> ... -> 1 (data-parallel degree
1 -> 2 -> ... -> N) and back up, through the relayout engine the runtime uses between ops whose layouts differ
(reference: `tensor_adapter`, runtime/megatron/mpu/mappings.py:382-468).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        benchmarks/reshard_bench.py [--tokens 16384] [--hidden 8192] [--iters 10] [--backend nccl|gloo]

Per transition one JSON line: bytes the busiest rank receives from other ranks, time (CUDA events on the GPU, max over ranks;
host clock on CPU), achieved GB/s per rank, the fraction of the measured NVLink peer bandwidth (770 GB/s per
direction), and the time of one NCCL all-to-all that moves the same number of bytes per rank (the collective a
tensor-parallel <-> data-parallel exchange maps to).  After the walk down and back up the tensor must equal the one
it started from; the last line says so.

With tensor-parallel degree t and data-parallel degree d a rank holds rows/d x hidden/t of the activation (rows split
over the data-parallel ranks, columns over the tensor-parallel ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 770.0   # measured peer copy per direction per GPU on this hardware generation's NVSwitch fabric


def _timed(fn, iters: int, cuda: bool) -> float:
    """Mean milliseconds per call, max over ranks."""
    fn()
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
    else:
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        ms = (time.perf_counter() - t0) * 1e3 / iters
    t = torch.tensor([ms], dtype=torch.float64, device="cuda" if cuda else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run(tokens: int, hidden: int, iters: int, dtype=torch.bfloat16, emit=print):
    from superscaler_b200.parallel.relayout import Layout, Side, local_shape, plan_transfer, relayout
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available() and dist.get_backend() == "nccl"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    assert world & (world - 1) == 0 and tokens % world == 0 and hidden % world == 0
    g = (tokens, hidden)
    degrees = []
    t = world
    while t >= 1:
        degrees.append((t, world // t))
        t //= 2
    walk = degrees + degrees[-2::-1]                      # tp N ... 1 ... N
    lay = lambda tp: Layout(row="split", col="split" if tp > 1 else "rep")   # noqa: E731
    gen = torch.Generator().manual_seed(7)
    full = torch.randn(g, generator=gen).to(dtype)

    def shard(tp, dp):
        side = Side(0, tp, dp)
        dr, tr = side.coords(rank)
        rows, cols = tokens // dp, hidden // tp
        return full[dr * rows:(dr + 1) * rows, tr * cols:(tr + 1) * cols].contiguous().to(dev)

    x = shard(*walk[0])
    esize = x.element_size()
    for (tp0, dp0), (tp1, dp1) in zip(walk, walk[1:]):
        src, dst = Side(0, tp0, dp0), Side(0, tp1, dp1)
        msgs = plan_transfer(src, lay(tp0), dst, lay(tp1), g, False)
        mine = sum((p.r1 - p.r0) * (p.c1 - p.c0) for m in msgs if m.dst == rank and m.src != rank for p in m.pieces) * esize
        r_t = torch.tensor([mine], dtype=torch.int64, device=dev)
        dist.all_reduce(r_t, op=dist.ReduceOp.MAX)       # ranks differ (some keep half of what they need, some nothing)
        recv = int(r_t.item())
        cur = x
        ms = _timed(lambda: relayout(cur, rank, src, lay(tp0), dst, lay(tp1)), iters, cuda)
        x = relayout(cur, rank, src, lay(tp0), dst, lay(tp1))
        assert tuple(x.shape) == tuple(local_shape(dst, lay(tp1), g))
        assert torch.equal(x.cpu(), shard(tp1, dp1).cpu()), f"rank {rank}: wrong shard after tp {tp0} -> {tp1}"
        # the same bytes per rank through one all-to-all
        n = max(world, recv // esize // world * world)
        a2a_in = torch.empty(n, dtype=dtype, device=dev)
        a2a_out = torch.empty_like(a2a_in)
        try:
            ms_a2a = _timed(lambda: dist.all_to_all_single(a2a_out, a2a_in), iters, cuda)
        except RuntimeError:                                   # a backend without all-to-all (gloo)
            ms_a2a = None
        if rank == 0:
            gbs = recv / ms / 1e6 if ms > 0 else 0.0
            emit(json.dumps({"case": "reshard", "from": f"tp{tp0}-dp{dp0}", "to": f"tp{tp1}-dp{dp1}", "tokens": tokens,
                             "hidden": hidden, "bytes_received_per_rank": recv, "ms": round(ms, 4),
                             "gbs_per_rank": round(gbs, 1), "nvlink_fraction": round(gbs / NVLINK_GBS, 3),
                             "nccl_all_to_all_ms": None if ms_a2a is None else round(ms_a2a, 4),
                             "timed_on": "device" if cuda else "host"}), flush=True)
    ok = torch.equal(x.cpu(), shard(*walk[0]).cpu())
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        emit(json.dumps({"round_trip_equal": bool(flag.item()), "transitions": len(walk) - 1}), flush=True)
    return bool(flag.item())


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--backend", default=None, choices=["nccl", "gloo"])
    a = ap.parse_args()
    backend = a.backend or ("nccl" if torch.cuda.is_available() else "gloo")
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend)
    ok = run(a.tokens, a.hidden, a.iters)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
