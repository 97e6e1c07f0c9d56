"""Where the device time of one training step goes: runs a committed plan for a few steps, records one step with
the CUDA activity tracer of torch.profiler and prints, per kernel, its share of the summed kernel time, launches and
mean duration, plus the fraction of the step's wall time during which some kernel ran ("busy"; well below 1 means
the host cannot issue launches fast enough).

    python -m superscaler_b200.profiler.step_breakdown --model {gpt,t5,resnet} [--plan plan.json] [--top 30]

A diagnostic, not a benchmark: the tracer adds overhead, so the step time printed here is not a throughput figure.
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import re
import time

import torch

PLANS = {"gpt": "gpt_1_3B_1gpu_b200.json", "t5": "t5_770M_1gpu_b200.json", "resnet": "resnet_1B_1gpu_b200.json"}


def _short(name: str) -> str:
    k = name.replace("(anonymous namespace)::", "").replace("void ", "")
    k = re.sub(r"\(.*", "", k)
    return re.sub(r"at::native::|at_cuda_detail::|std::array<char\*, \d+ul> ?", "", k)[:100]


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="gpt", choices=sorted(PLANS))
    ap.add_argument("--plan", default=None, help="plan JSON (default: the committed 1-GPU plan of the model)")
    ap.add_argument("--top", type=int, default=30)
    a = ap.parse_args(argv)
    from torch.profiler import ProfilerActivity, profile

    from ..data import synthetic
    from ..runtime.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    with open(a.plan or os.path.join(root, "plans", PLANS[a.model])) as f:
        plan = json.load(f)
    tr = Trainer(plan, rank=0, world_size=1, model_overrides=dict(vocab=51200) if a.model == "gpt" else {})
    cfg, gbs = tr.cfg, plan["global_batch_size"]
    if a.model == "t5":
        batch = synthetic.t5_batch(gbs, cfg.seq_length, cfg.dec_seq_length, cfg.vocab, seed=1)
    elif a.model == "gpt":
        batch = synthetic.gpt_batch(gbs, plan["seq_length"], 51200, seed=1)
    else:
        batch = synthetic.resnet_batch(gbs, cfg.image_size, cfg.num_classes, seed=1)
    batch = tr.to_device(batch)
    for _ in range(2):
        tr.train_step(batch)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tr.train_step(batch)
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        tr.train_step(batch)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    total = sum(e.device_time for e in ev) / 1e3
    print(f"{a.model}: untraced step {wall:.1f} ms, {len(ev)} device activities, summed kernel time {total:.1f} ms, "
          f"busy {total / wall:.2f}")
    ms, n = collections.Counter(), collections.Counter()
    for e in ev:
        k = _short(e.name)
        ms[k] += e.device_time / 1e3
        n[k] += 1
    for k, v in ms.most_common(a.top):
        print(f"  {v / total * 100:5.1f}% {v:9.1f} ms {n[k]:6d} x {v / n[k] * 1e3:8.1f} us  {k}")


if __name__ == "__main__":
    main()
