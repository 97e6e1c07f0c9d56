"""Checks and timings of the fused compute + collective kernels against the NCCL path, callable from `bench.py`
(untimed self-check before its timed regions on 2 or more GPUs) and from benchmarks/fused_collective_bench.py.

  self_check : GEMM -> all-reduce, GEMM -> reduce-scatter and all-gather -> GEMM in one kernel each against the same
               GEMM with an NCCL collective, on two shapes; maximum relative error and the kernels' status word.
  microbench : the resharding / fused-collective micro-benchmark: activations [mbs x 2048 tokens, hidden] in bf16 with
               [hidden, 4 hidden] weights at tensor-parallel degree = the number of ranks,
                 all-gather -> GEMM  (rows dealt out over the ranks -> column-parallel up-projection: dp -> tp)
                 GEMM -> reduce-scatter (its backward, and tp -> dp after a row-parallel down-projection)
                 GEMM -> all-reduce  (row-parallel down-projection that stays tensor parallel)
               each as fused time, NCCL-path time, NVLink bytes per GPU, achieved GB/s and fraction of the roofline
               max(FLOPs / measured GEMM rate, bytes / measured link bandwidth).
All times are CUDA events on the launching stream after warm-up, maximum over the ranks.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch
import torch.distributed as dist

LINK_GBS = 770.0          # measured peer-copy bandwidth per direction per GPU on this machine class


def gemm_peak_tflops() -> tuple:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f).get("bf16_tflops", 1590.0)), "measured"
    except Exception:  # noqa: BLE001 - no measurement file: the stated fallback
        return 1590.0, "fallback"


_L2_FLUSH = None


def _timed(fn, warmup: int, iters: int) -> float:
    """Mean device time of one call (CUDA events around every call, max over ranks).  Between calls a 256 MB buffer
    is overwritten, outside the timed span, so that operands come from HBM and not from the 126 MB L2."""
    global _L2_FLUSH
    if _L2_FLUSH is None:
        _L2_FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    pairs = []
    for _ in range(iters):
        _L2_FLUSH.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        pairs.append((e0, e1))
    torch.cuda.synchronize()
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in pairs) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9))


def self_check(ctx, dev, rank: int, world: int) -> Dict[str, float]:
    """Maximum relative error of the three fused kernels against GEMM + NCCL, on two shapes each."""
    from ..ops import functional as F, native
    out = {"gemm_allreduce": 0.0, "gemm_reduce_scatter": 0.0, "allgather_gemm": 0.0}
    for (M, N, K) in ((256 * world, 512, 256), (2048, 2048, 1024)):
        g = torch.Generator(device=dev).manual_seed(17 * rank + M)
        x = (torch.randn(M, K, device=dev, generator=g) * 0.5).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.1).bfloat16()
        y = F.gemm(x, w, out_dtype=torch.float32)
        rs_ref = torch.empty(M // world, N, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(rs_ref, y.clone())
        dist.all_reduce(y)
        out["gemm_allreduce"] = max(out["gemm_allreduce"], _rel(ctx.linear_allreduce(x, w), y))
        out["gemm_reduce_scatter"] = max(out["gemm_reduce_scatter"], _rel(ctx.linear_reduce_scatter(x, w), rs_ref))
        rows = M // world
        xs = x[:rows].contiguous()
        g2 = torch.Generator(device=dev).manual_seed(5 + M)                 # the same weight on every rank
        w2 = (torch.randn(N, K, device=dev, generator=g2) * 0.05).bfloat16()
        ctx.ensure_allgather(M, K)
        full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, xs)
        out["allgather_gemm"] = max(out["allgather_gemm"], _rel(ctx.allgather_linear(xs, w2), F.gemm(full, w2)))
    torch.cuda.synchronize()
    out["kernel_status"] = native.check_status()
    out["passed"] = bool(out["kernel_status"] == 0 and max(out["gemm_allreduce"], out["gemm_reduce_scatter"],
                                                           out["allgather_gemm"]) < 2e-2)
    return out


def microbench(ctx, dev, rank: int, world: int, mbs_list=(1, 8), hidden_list=(2048, 8192), seq: int = 2048,
               warmup: int = 3, iters: int = 10) -> List[dict]:
    from ..ops import functional as F, native
    peak_tf, peak_src = gemm_peak_tflops()
    rows_out: List[dict] = []

    def finish(row, fused_ms, nccl_ms, flops, nv_bytes):
        t_flops = flops / (peak_tf * 1e12) * 1e3
        t_link = nv_bytes / (LINK_GBS * 1e9) * 1e3
        row.update(fused_ms=round(fused_ms, 4), nccl_path_ms=round(nccl_ms, 4), nvlink_bytes_per_gpu=int(nv_bytes),
                   fused_gbs=round(nv_bytes / fused_ms / 1e6, 1), roofline_ms=round(max(t_flops, t_link), 4),
                   roofline_fraction=round(max(t_flops, t_link) / fused_ms, 3),
                   speedup_vs_nccl_path=round(nccl_ms / fused_ms, 3), gemm_peak=f"{peak_tf} TFLOP/s ({peak_src})")
        rows_out.append(row)

    for h in hidden_list:
        for mbs in mbs_list:
            M = mbs * seq
            if not ctx.fits(M, h) or (M // world) % 128:
                continue
            g = torch.Generator(device=dev).manual_seed(1234 + rank)
            # ---- row-parallel down-projection: [M, 4h / tp] x [h, 4h / tp]^T, summed over the ranks ----
            K = 4 * h // world
            x = torch.randn(M, K, device=dev, generator=g).bfloat16()
            w = (torch.randn(h, K, device=dev, generator=g) * 0.02).bfloat16()
            out_ar = torch.empty(M, h, device=dev, dtype=torch.bfloat16)
            out_rs = torch.empty(M // world, h, device=dev, dtype=torch.bfloat16)
            flops = 2.0 * M * h * K

            def nccl_ar():
                y = F.gemm(x, w)
                dist.all_reduce(y)
                return y

            def nccl_rs():
                y = F.gemm(x, w)
                dist.reduce_scatter_tensor(out_rs, y)

            t_f = _timed(lambda: ctx.linear_allreduce(x, w, out=out_ar), warmup, iters)
            finish({"case": "gemm_allreduce", "tp": world, "M": M, "N": h, "K_per_rank": K}, t_f,
                   _timed(nccl_ar, warmup, iters), flops, 2 * (world - 1) / world * M * h * 2)
            t_f = _timed(lambda: ctx.linear_reduce_scatter(x, w, out=out_rs), warmup, iters)
            finish({"case": "gemm_reduce_scatter", "tp": world, "M": M, "N": h, "K_per_rank": K}, t_f,
                   _timed(nccl_rs, warmup, iters), flops, (world - 1) / world * M * h * 2)
            # ---- column-parallel up-projection on rows dealt out over the ranks: gather [M, h], x [4h / tp, h]^T ----
            N = 4 * h // world
            xs = torch.randn(M // world, h, device=dev, generator=g).bfloat16()
            w_up = (torch.randn(N, h, device=dev, generator=g) * 0.02).bfloat16()
            full = torch.empty(M, h, device=dev, dtype=torch.bfloat16)
            out_ag = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            ctx.ensure_allgather(M, h)

            def nccl_ag():
                dist.all_gather_into_tensor(full, xs)
                return F.gemm(full, w_up, out_ag)

            t_f = _timed(lambda: ctx.allgather_linear(xs, w_up, out=out_ag), warmup, iters)
            finish({"case": "allgather_gemm", "tp": world, "M": M, "N_per_rank": N, "K": h}, t_f,
                   _timed(nccl_ag, warmup, iters), 2.0 * M * N * h, (world - 1) / world * M * h * 2)
    for r in rows_out:
        r["kernel_status"] = native.check_status()
    return rows_out


def run_in_bench(dev, rank: int, world: int, max_mbs: int = 8, max_hidden: int = 8192) -> dict:
    """The untimed block `bench.py` runs on 2 or more GPUs before its timed regions."""
    from ..parallel.symm import FusedTPContext
    ctx = FusedTPContext(None, max_mbs * 2048, max_hidden, dev)
    out = {"self_check": self_check(ctx, dev, rank, world)}
    out["microbench"] = microbench(ctx, dev, rank, world, mbs_list=(1, max_mbs), hidden_list=(2048, max_hidden))
    del ctx
    torch.cuda.empty_cache()
    return out
