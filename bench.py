"""Headline benchmark: GPT-3 1.3B training throughput (samples/s) at global batch 512 on N B200 GPUs.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...            # the unmodified reference (when installable)

For N > 1 launch one rank per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Model / config (fixed): 24 layers, hidden 2048, 16 heads x 128, FFN 8192 GeLU, pre-LayerNorm, seq 2048,
vocab 51200, bf16 weights N(0, 0.02), dropout 0.1 (hidden and attention), Adam + clip 1.0, global batch 512;
token ids uniform over [0, 51200) from a seed (synthetic).  Strong scaling: the global batch stays 512.
`--model t5` / `--model resnet` run the other two model families of the reference's evaluation (T5 770M at global
batch 512, Wide-ResNet 1B at global batch 768) through the same two timed regions with their committed plans.

Two timed regions, W warm-up steps before each, K steps inside, CUDA events bracketed by barrier +
synchronize, max over ranks:
  value : inputs already resident on the device, no host read inside the region;
  e2e   : the public API end to end -- every step copies that step's batch from pinned host memory and reads
          the step's loss back to the host.
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

PUBLISHED_BASELINE = 8.68  # samples/s, GPT-3 1.3B, GBS 512, reference's published 4-GPU searched plan

GPT13B = dict(num_layers=24, hidden_size=2048, num_attention_heads=16, kv_channels=128, ffn_hidden_size=8192,
              seq_length=2048, max_position_embeddings=2048, vocab_size=51200)
GLOBAL_BS = 512


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt", choices=["gpt", "t5", "resnet"],
                    help="gpt (default, the headline): GPT-3 1.3B, global batch 512; t5: T5 770M (encoder 512 / decoder "
                         "128 tokens, ReLU, relative-position buckets), global batch 512; resnet: Wide-ResNet 1B, global "
                         "batch 768 -- each with the committed searched plan for N GPUs")
    ap.add_argument("--mbs-per-gpu", type=int, default=8)
    ap.add_argument("--plan", default=None, help="plan JSON (default: the committed searched plan for N GPUs, "
                                                 "else pure data parallel)")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BS)
    ap.add_argument("--layers", type=int, default=None, help="debug only; a non-default value is reported")
    ap.add_argument("--fused-comm", type=int, default=1)
    ap.add_argument("--fused-check", type=int, default=1,
                    help="on 2 or more GPUs: check and time the fused GEMM + collective kernels against the NCCL path "
                         "before the timed regions (reported under 'fused_collectives')")
    ap.add_argument("--deterministic", type=int, default=0,
                    help="1: bitwise-reproducible kernels (attention backward as the dK/dV + dQ kernel pair)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, mx, reasons, power = [], None, set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                clocks.append(float(f[1]))
                mx = float(f[2])
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": mx,
                "power_w_max": max(power) if power else None, "samples": len(clocks), "reasons": sorted(reasons)}


def default_plan(n_gpus: int, mbs_per_gpu: int, global_bs: int, layers: int) -> dict:
    from superscaler_b200.models.gpt import gpt_op_names
    here = os.path.dirname(os.path.abspath(__file__))
    searched = os.path.join(here, "plans", f"gpt_1_3B_{n_gpus}gpu_b200.json")
    if os.path.exists(searched) and layers == GPT13B["num_layers"] and global_bs == GLOBAL_BS:
        with open(searched) as f:
            return json.load(f)
    n = len(gpt_op_names(layers))
    d = dict(model_name="gpt", model_size="1_3B", **GPT13B)
    d["num_layers"] = layers
    d.update(global_batch_size=global_bs, micro_batch_size=mbs_per_gpu * n_gpus, num_stages=1, num_gpus=[n_gpus],
             checkpoint_activations=[False], resharding_stages=[False], num_ops_in_each_stage=[n],
             model_parallel_size_of_each_op=[[1] * n], data_parallel_size_of_each_op=[[n_gpus] * n],
             recompute_ops=[[0] * n], algo_of_each_op=[[0] * n])
    return d


def describe_parallelism(plan: dict) -> str:
    tps = sorted({t for s in plan["model_parallel_size_of_each_op"] for t in s})
    dps = sorted({t for s in plan["data_parallel_size_of_each_op"] for t in s})
    return f"pp{plan['num_stages']}-tp{'/'.join(map(str, tps))}-dp{'/'.join(map(str, dps))}-mbs{plan['micro_batch_size']}"


def run_reference(args):
    """The unmodified reference on the same metric and config; rank 0 prints the one JSON line."""
    from baseline import reference_arm
    rank = int(os.environ.get("RANK", "0"))
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 else None
    if sampler:
        sampler.start()
    out = reference_arm.run(args)
    if sampler:
        clocks = sampler.stop()
        if "unavailable" not in out:
            out["clocks"] = clocks
    if rank == 0:
        print(json.dumps(out), flush=True)
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001 - the line is printed; a failed teardown must not change the exit code
        pass


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist

    from superscaler_b200.data.synthetic import gpt_batch
    from superscaler_b200.ops import native
    from superscaler_b200.parallel.state import init_distributed
    from superscaler_b200.runtime.trainer import Trainer

    rank, world, local = init_distributed()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    layers = args.layers or GPT13B["num_layers"]
    here = os.path.dirname(os.path.abspath(__file__))
    if args.plan:
        with open(args.plan) as f:
            plan = json.load(f)
    elif args.model == "gpt":
        plan = default_plan(world, args.mbs_per_gpu, args.global_batch, layers)
    else:
        name = {"t5": "t5_770M", "resnet": "resnet_1B"}[args.model]
        with open(os.path.join(here, "plans", f"{name}_{world}gpu_b200.json")) as f:
            plan = json.load(f)
    if args.deterministic:
        from superscaler_b200.ops import functional as F
        F.set_deterministic(True)
    overrides = dict(vocab=GPT13B["vocab_size"]) if args.model == "gpt" else {}
    trainer = Trainer(plan, rank=rank, world_size=world, fused_comm=bool(args.fused_comm), model_overrides=overrides)
    gbs = plan["global_batch_size"]
    cfg = trainer.cfg
    if args.model == "gpt":
        seq, vocab = plan["seq_length"], GPT13B["vocab_size"]
        make_batch = lambda seed: gpt_batch(gbs, seq, vocab, seed=seed)
        metric = "samples/s (GPT-3 1.3B, GBS 512, searched plan)"
        model_desc = "GPT-3 1.3B (24L, h2048, 16x128 heads, ffn 8192, seq 2048, vocab 51200, dropout 0.1)"
        data_desc = "synthetic (token ids uniform over [0, 51200) from a seed; random-init weights)"
        published = PUBLISHED_BASELINE
    elif args.model == "t5":
        from superscaler_b200.data.synthetic import t5_batch
        seq = cfg.seq_length
        make_batch = lambda seed: t5_batch(gbs, cfg.seq_length, cfg.dec_seq_length, cfg.vocab, seed=seed)
        metric = "samples/s (T5 770M, GBS 512, searched plan)"
        model_desc = (f"T5 770M ({cfg.num_layers}+{cfg.num_layers}L, d_model {cfg.hidden}, {cfg.heads}x{cfg.head_dim} heads, "
                      f"d_ff {cfg.ffn} ReLU, relative-position buckets {cfg.relative_attention_num_buckets if cfg.relative_position_bias else 0}, "
                      f"vocab {cfg.vocab}, encoder {cfg.seq_length} / decoder {cfg.dec_seq_length} tokens)")
        data_desc = "synthetic (token ids uniform from a seed; random-init weights)"
        published = 15.14      # reference README.md:132, 4 unnamed GPUs
    else:
        from superscaler_b200.data.synthetic import resnet_batch
        seq = cfg.image_size
        make_batch = lambda seed: resnet_batch(gbs, cfg.image_size, cfg.num_classes, seed=seed)
        metric = "samples/s (Wide-ResNet 1B, GBS 768, searched plan)"
        model_desc = (f"Wide-ResNet 1B (bottleneck ResNet-50 layout, base channels {plan['in_channels']}, width factor "
                      f"{plan['width_factor']}, {cfg.num_classes} classes, {cfg.image_size}x{cfg.image_size}x3 images)")
        data_desc = "synthetic (images N(0,1), labels uniform, from a seed; Kaiming random-init weights)"
        published = 41.52      # reference README.md:135, 4 unnamed GPUs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    verbose = os.environ.get("SSB_BENCH_VERBOSE") == "1" and rank == 0

    host_issue_ms = [0.0]

    def timed(step_fn, n_warm, n_steps):
        for i in range(n_warm):
            t_w = time.perf_counter()
            step_fn(i)
            if verbose:
                torch.cuda.synchronize()
                print(f"[bench] warm-up step {i}: {time.perf_counter() - t_w:.2f} s", file=sys.stderr, flush=True)
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        native.launch_counter["kernels"] = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for i in range(n_steps):
            step_fn(n_warm + i)
        e1.record()
        enqueue = (time.perf_counter() - t0) * 1000.0      # host time to issue the steps (the device runs behind)
        barrier()
        wall = (time.perf_counter() - t0) * 1000.0
        clocks = sampler.stop()
        ms = torch.tensor([e0.elapsed_time(e1), wall, enqueue], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        host_issue_ms[0] = ms[2].item() / n_steps
        return ms[0].item() / n_steps, ms[1].item() / n_steps, clocks, native.launch_counter["kernels"]

    # ---- 2 or more GPUs: the fused compute + collective kernels against the NCCL path (untimed) --------------
    fused = None
    if world > 1 and args.fused_check:
        try:
            from superscaler_b200.profiler import fused_bench
            fused = fused_bench.run_in_bench(torch.device("cuda", local), rank, world)
        except Exception as e:  # noqa: BLE001 - reported in the JSON line, the training benchmark goes on
            fused = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
        barrier()

    # ---- device-timed region: batches resident on the device ----------------------------------
    resident = [trainer.to_device(make_batch(1000 + i)) for i in range(2)]

    def step_resident(i):
        trainer.train_step(resident[i % 2])

    ms_dev, _, clocks, launches = timed(step_resident, args.warmup, args.steps)
    issue_dev = host_issue_ms[0]
    del resident

    # ---- end-to-end region: pinned host batch -> device every step, loss read back every step ---
    host = [make_batch(2000 + i) for i in range(2)]
    last_loss = [0.0]

    def step_e2e(i):
        stats = trainer.train_step(host[i % 2])
        last_loss[0] = trainer.loss_value(stats)

    ms_e2e, wall_e2e, clocks_e2e, _ = timed(step_e2e, max(1, min(args.warmup, 3)), args.steps)
    h2d = sum(t.numel() * t.element_size() for t in host[0].values())
    status = native.check_status()

    if rank == 0:
        value = gbs / (ms_dev / 1000.0)
        e2e_value = gbs / (max(ms_e2e, wall_e2e) / 1000.0)
        out = {
            "metric": metric, "value": round(value, 3), "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_dev, 2),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": round(value / published, 3),
            "dtype": "bf16", "data": data_desc,
            "impl": "ours",
            "config": {"model": model_desc,
                       "global_batch": gbs, "seq_len": seq, "parallelism": describe_parallelism(plan),
                       "num_microbatches": trainer.num_microbatches, "l2": "inputs_exceed_l2 (2.6 GB of weights + "
                       "activations stream through every step)", "layers": layers if args.model == "gpt" else plan["num_layers"],
                       "params": trainer.num_parameters(), "host_issue_ms_per_step": round(issue_dev, 2), "kernel_status": status, "last_loss": round(last_loss[0], 4),
                       "max_allocated_mb": round(torch.cuda.max_memory_allocated() / 2 ** 20)},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 3), "unit": "samples/s", "ms_per_step": round(max(ms_e2e, wall_e2e), 2),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "clocks": clocks_e2e},
            "gpu_launches": launches,
        }
        if fused is not None:
            out["fused_collectives"] = fused
        if args.model == "gpt" and (layers != GPT13B["num_layers"] or gbs != GLOBAL_BS):
            out["invalid_reduced_config"] = True
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
