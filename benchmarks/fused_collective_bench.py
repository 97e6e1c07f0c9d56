"""Fused compute + collective micro-benchmark.

  gemm_allreduce : GEMM -> all-reduce in one kernel (csrc/gemm_ar_sm100.cu) against the same GEMM followed by an
                   NCCL all-reduce and the bias / dropout / residual kernel;
  allgather_gemm : all-gather -> GEMM in one kernel (csrc/gemm_ag_sm100.cu) against an NCCL all-gather followed by
                   the same GEMM (activations [mbs x 2048 / tp rows per rank, hidden] times [4 x hidden / tp, hidden]).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/fused_collective_bench.py [--mbs 1 4 8] [--hidden 2048 4096 8192] [--iters 20]

Shapes: activations [mbs x 2048 tokens, 4 x hidden / tp] times the row-parallel weight [hidden, 4 x hidden / tp]
(the MLP down-projection of a tensor-parallel transformer layer).  Per case rank 0 prints one JSON line with the
device time of both paths (CUDA events, max over ranks, after warm-up), the bytes every GPU must move over
NVLink for a two-shot all-reduce (2 (tp-1)/tp M N 2 B), the achieved GB/s of the fused kernel counted on those
bytes, and the roofline fraction: max(FLOPs / measured GEMM peak, bytes / link bandwidth) / fused time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS = 770.0          # measured peer-copy bandwidth per direction per GPU on this machine class


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops", 1590.0)), "measured"
    except Exception:  # noqa: BLE001
        return 1590.0, "fallback"


def timed(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mbs", type=int, nargs="+", default=[1, 4, 8])
    ap.add_argument("--hidden", type=int, nargs="+", default=[2048, 4096, 8192])
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    from superscaler_b200.ops import functional as F, native
    from superscaler_b200.parallel.state import init_distributed
    from superscaler_b200.parallel.symm import FusedTPContext
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    peak_tf, peak_src = peaks()
    ctx = FusedTPContext(None, max(a.mbs) * a.seq, max(a.hidden), dev)
    for h in a.hidden:
        for mbs in a.mbs:
            M, N, K = mbs * a.seq, h, 4 * h // world
            g = torch.Generator(device=dev).manual_seed(1234 + rank)
            x = torch.randn(M, K, device=dev, generator=g).bfloat16()
            w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
            bias = torch.zeros(N, device=dev, dtype=torch.bfloat16)
            res = torch.randn(M, N, device=dev, generator=g).bfloat16()
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

            def nccl_path():
                y = F.gemm(x, w)
                dist.all_reduce(y)
                return F.bias_dropout_add(y, bias, res, 0.1, 7)

            def gemm_only():
                return F.gemm(x, w)

            row = {"case": "gemm_allreduce", "tp": world, "M": M, "N": N, "K_per_rank": K}
            row["gemm_only_ms"] = timed(gemm_only, a.warmup, a.iters)
            row["nccl_path_ms"] = timed(nccl_path, a.warmup, a.iters)
            for name in ("fused_ms",):
                row[name] = timed(lambda: ctx.linear_allreduce(x, w, bias=bias, residual=res, dropout_p=0.1, seed=7,
                                                               out=out), a.warmup, a.iters)
            best = min(v for k, v in row.items() if k.startswith("fused_"))
            nv_bytes = 2 * (world - 1) / world * M * N * 2
            t_flops = 2 * M * N * K / (peak_tf * 1e12) * 1e3
            t_link = nv_bytes / (LINK_GBS * 1e9) * 1e3
            row.update(nvlink_bytes_per_gpu=int(nv_bytes), fused_gbs=nv_bytes / best / 1e6,
                       roofline_ms=max(t_flops, t_link), roofline_fraction=max(t_flops, t_link) / best,
                       speedup_vs_nccl_path=row["nccl_path_ms"] / best, gemm_peak=f"{peak_tf} TFLOP/s ({peak_src})",
                       kernel_status=native.check_status())
            if rank == 0:
                print(json.dumps(row), flush=True)
    # ---- all-gather -> GEMM -----------------------------------------------------------------------------
    ctx.enable_allgather(max(a.mbs) * a.seq, max(a.hidden))
    for h in a.hidden:
        for mbs in a.mbs:
            M, N, K = mbs * a.seq, 4 * h // world, h
            if (M // world) % 128:
                continue
            g = torch.Generator(device=dev).manual_seed(99 + rank)
            x = torch.randn(M // world, K, device=dev, generator=g).bfloat16()
            w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
            bias = torch.zeros(N, device=dev, dtype=torch.bfloat16)
            full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

            def nccl_path():
                dist.all_gather_into_tensor(full, x)
                return F.gemm(full, w, out, bias=bias, act=F.ACT_GELU)

            row = {"case": "allgather_gemm", "tp": world, "M": M, "N_per_rank": N, "K": K}
            row["gemm_only_ms"] = timed(lambda: F.gemm(full, w, out, bias=bias, act=F.ACT_GELU), a.warmup, a.iters)
            row["nccl_path_ms"] = timed(nccl_path, a.warmup, a.iters)
            row["fused_ms"] = timed(lambda: ctx.allgather_linear(x, w, bias=bias, act=F.ACT_GELU, out=out), a.warmup,
                                    a.iters)
            nv_bytes = (world - 1) / world * M * K * 2          # received (and sent) per GPU
            t_flops = 2 * M * N * K / (peak_tf * 1e12) * 1e3
            t_link = nv_bytes / (LINK_GBS * 1e9) * 1e3
            row.update(nvlink_bytes_per_gpu=int(nv_bytes), fused_gbs=nv_bytes / row["fused_ms"] / 1e6,
                       roofline_ms=max(t_flops, t_link), roofline_fraction=max(t_flops, t_link) / row["fused_ms"],
                       speedup_vs_nccl_path=row["nccl_path_ms"] / row["fused_ms"],
                       gemm_peak=f"{peak_tf} TFLOP/s ({peak_src})", kernel_status=native.check_status())
            if rank == 0:
                print(json.dumps(row), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
