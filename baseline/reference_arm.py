"""`bench.py --impl reference`: the reference's own runtime on the same metric and config.

The unmodified reference tree (runtime/, search/, profiler/) sits under baseline/_ref (copied there by
`__graft_entry__.build()`; the directory is not tracked).  This module is the launcher around it and never edits it:

* the reference imports NVIDIA apex (runtime/megatron/optimizer/__init__.py:16-17, optimizer/clip_grads.py:21-22,
  optimizer/optimizer.py:23-24, utils.py:31-32), which is not in this image: baseline/shims/ holds stand-in `apex`
  and `amp_C` modules built on torch's fused multi-tensor kernels and is put on sys.path;
* `torch._six` (optimizer/clip_grads.py:19) left torch in 2.0: a module object with `inf` and `string_classes` is
  registered in sys.modules before the reference is imported;
* numpy dropped the `np.float` / `np.int` aliases that runtime/megatron/data/indexed_dataset.py:98 names at import
  time: the aliases are set on the numpy module;
* the reference JIT-builds its four CUDA extensions with explicit sm_70 / sm_80 flags
  (runtime/megatron/fused_kernels/__init__.py:30-95); with a GPU present torch's extension builder adds the flags of
  the visible device by itself, and NVCC_APPEND_FLAGS adds sm_100 as well, so the same sources also carry Blackwell
  code;
* the plan JSON is written here in the reference's schema (runtime/megatron/arguments.py:90-124) for the benchmark's
  model: GPT-3 1.3B with 24 layers, hidden 2048, 16 heads, sequence 2048, global batch 512, one stage, data parallel
  over all GPUs; `--make-vocab-size-divisible-by 1024` pads GPT-2's 50257 tokens to exactly 51200;
* the command line is the stock one of runtime/scripts/run_gpt.sh:22-43, run in this process (one process per GPU,
  RANK / WORLD_SIZE / MASTER_* from the environment) through `runpy`.

The time is the reference's own: "elapsed time per iteration (ms)" of its training log
(runtime/megatron/training.py:858-895, the value its per-rank CSV stores at :903-908), one value per iteration; the
first `warmup` iterations are dropped and the mean of the following `steps` is reported.  The reference creates its
batches on the device inside `get_batch` (runtime/pretrain_gpt.py:50-62) and reads the loss back every iteration,
so its iteration time is its end-to-end time.
"""
from __future__ import annotations

import io
import json
import os
import re
import sys
import tempfile
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
RUNTIME = os.path.join(REF, "runtime")
SHIMS = os.path.join(HERE, "shims")
PREBUILT_MARK = os.path.join(REF, ".prebuilt_runtime_path")


def runtime_dir() -> str:
    """The reference's runtime directory, spelled the way it was when its extensions were pre-built: ninja keys its
    up-to-date check on absolute source paths, so another spelling of the same directory (a symlinked checkout) would
    make the reference's loader compile everything again."""
    try:
        with open(PREBUILT_MARK) as f:
            recorded = f.read().strip()
        if recorded and os.path.samefile(recorded, RUNTIME):
            return recorded
    except OSError:
        pass
    return RUNTIME

PUBLISHED_SAMPLES_PER_S = 8.68          # README.md:129 of the reference (4 unnamed GPUs)
GPT_LAYER_OPS = 13                      # runtime/megatron/model/flex_gpt.py:18-41

# (per-GPU micro-batch, recompute every transformer layer?) tried for the reference on a B200; the reference keeps the
# [b, heads, s, s] attention scores of every layer (about 0.6 GB per sample and layer), so without recompute its
# micro-batch is bounded by memory.  The entry used by default is the fastest of the grid measured on one B200.
REFERENCE_GRID = ((4, False), (8, False), (16, True))
DEFAULT_MICRO_BATCH = 8
DEFAULT_RECOMPUTE = False


def gpt_plan(n_gpus: int, micro_batch_per_gpu: int, recompute: bool, layers: int = 24, hidden: int = 2048,
             heads: int = 16, seq: int = 2048, global_batch: int = 512) -> dict:
    """One-stage data-parallel plan in the reference's JSON schema (search/aceso_utils.py:137-211)."""
    n_ops = 1 + GPT_LAYER_OPS * layers + 2
    rec = [0] + ([1] * GPT_LAYER_OPS * layers if recompute else [0] * GPT_LAYER_OPS * layers) + [0, 0]
    return {
        "model_name": "gpt", "model_size": "1_3B", "num_layers": layers, "seq_length": seq,
        "max_position_embeddings": seq, "num_attention_heads": heads, "hidden_size": hidden,
        "global_batch_size": global_batch, "micro_batch_size": micro_batch_per_gpu * n_gpus, "num_stages": 1,
        "num_gpus": [n_gpus], "checkpoint_activations": [bool(recompute)], "resharding_stages": [False],
        "num_ops_in_each_stage": [n_ops], "model_parallel_size_of_each_op": [[1] * n_ops],
        "data_parallel_size_of_each_op": [[n_gpus] * n_ops], "recompute_ops": [rec], "algo_of_each_op": [[0] * n_ops],
    }


def stock_argv(plan_path: str, log_path: str, train_iters: int, dtype: str) -> list:
    """The command line of runtime/scripts/run_gpt.sh:22-43 (paths filled in, iteration count from the caller)."""
    return ["pretrain_gpt.py",
            "--flexpipe-config", plan_path,
            "--train-iters", str(train_iters),
            "--eval-iters", "0",
            "--lr-decay-iters", "320000",
            "--vocab-file", "vocabs/gpt2-vocab.json",
            "--merge-file", "vocabs/gpt2-merges.txt",
            "--data-impl", "mmap",
            "--split", "949,50,1",
            "--distributed-backend", "nccl",
            "--lr", "0.00015",
            "--lr-decay-style", "cosine",
            "--min-lr", "1.0e-5",
            "--weight-decay", "1e-2",
            "--clip-grad", "1.0",
            "--lr-warmup-fraction", ".01",
            "--log-interval", "1",
            "--DDP-impl", "local",
            "--" + dtype,
            "--make-vocab-size-divisible-by", "1024",
            "--log-path", log_path]


class _Tee(io.TextIOBase):
    def __init__(self, stream, sink):
        self.stream, self.sink = stream, sink

    def write(self, s):
        self.sink.append(s)
        return self.stream.write(s)

    def flush(self):
        self.stream.flush()


def _install_shims() -> None:
    six = types.ModuleType("torch._six")
    six.inf = float("inf")
    six.string_classes = (str, bytes)
    sys.modules["torch._six"] = six
    import torch
    torch._six = six
    import numpy
    for alias, target in (("float", float), ("int", int), ("bool", bool), ("object", object), ("str", str)):
        if alias not in numpy.__dict__:                  # aliases removed in numpy 1.24 (data/indexed_dataset.py:98)
            setattr(numpy, alias, target)
    # torch's extension loader no longer registers a JIT-built module in sys.modules, while the reference imports its
    # extensions by name afterwards (model/fused_layer_norm.py:68, model/fused_softmax.py:32-105): its own build
    # directory goes on the module search path
    built = os.path.join(runtime_dir(), "megatron", "fused_kernels", "build")
    if built not in sys.path:
        sys.path.append(built)
    for p in (runtime_dir(), SHIMS):
        if p not in sys.path:
            sys.path.insert(0, p)
    flags = os.environ.get("NVCC_APPEND_FLAGS", "")
    if "sm_100" not in flags:
        os.environ["NVCC_APPEND_FLAGS"] = (flags + " -gencode arch=compute_100,code=sm_100").strip()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")


def parse_iteration_times(text: str) -> list:
    """Milliseconds per iteration from the reference's log lines (runtime/megatron/training.py:861-865)."""
    return [float(m) for m in re.findall(r"elapsed time per iteration \(ms\): ([0-9.]+)", text)]


def run(args) -> dict:
    import torch
    if getattr(args, "model", "gpt") != "gpt":
        return {"impl": "reference", "unavailable": f"the reference arm runs the headline model (GPT-3 1.3B) only, not "
                                                    f"--model {args.model}"}
    if not os.path.isfile(os.path.join(RUNTIME, "pretrain_gpt.py")):
        return {"impl": "reference", "unavailable": "no reference tree under baseline/_ref (run __graft_entry__.build())"}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "the reference runtime needs a CUDA device (it calls .cuda() and "
                "NCCL unconditionally); none is visible"}
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        return {"impl": "reference", "unavailable": f"launched with WORLD_SIZE {world} but --gpus {args.gpus}: start "
                "the reference arm with one process per GPU (torch.distributed.run), as the own arm is"}
    mbs = int(os.environ.get("SSB_REF_MICRO_BATCH", DEFAULT_MICRO_BATCH))
    recompute = os.environ.get("SSB_REF_RECOMPUTE", "1" if DEFAULT_RECOMPUTE else "0") == "1"
    dtype = os.environ.get("SSB_REF_DTYPE", "bf16")
    while 512 % (mbs * world):
        mbs //= 2
    steps, warmup = args.steps, max(args.warmup, 1)

    work = os.environ.get("SSB_REF_WORKDIR") or os.path.join(tempfile.gettempdir(), "ssb_reference_arm")
    log_path = os.path.join(work, "logs") + "/"
    os.makedirs(os.path.join(log_path, "csv"), exist_ok=True)
    plan_path = os.path.join(work, f"gpt_1_3B_dp{world}_mbs{mbs}_rank{rank}.json")
    with open(plan_path, "w") as f:
        json.dump(gpt_plan(world, mbs, recompute), f)

    _install_shims()
    import runpy
    captured: list = []
    old = (sys.argv, os.getcwd(), sys.stdout)
    sys.argv = stock_argv(plan_path, log_path, warmup + steps, dtype)
    os.chdir(runtime_dir())
    sys.stdout = _Tee(old[2], captured)
    error = None
    try:
        runpy.run_path(os.path.join(runtime_dir(), "pretrain_gpt.py"), run_name="__main__")
    except SystemExit as e:                                  # the reference leaves through sys.exit in places
        if e.code not in (None, 0):
            error = f"reference exited with code {e.code}"
    except Exception as e:                                   # noqa: BLE001 - reported as the unavailable reason
        error = f"{type(e).__name__}: {str(e)[:300]}"
    finally:
        sys.stdout.flush()
        sys.argv, _, sys.stdout = old
        os.chdir(old[1])
    if error is not None:
        return {"impl": "reference", "unavailable": "the reference runtime failed on this box: " + error}

    # only the last rank prints the log line; bring its numbers to every rank
    times = parse_iteration_times("".join(captured))
    import torch.distributed as dist
    if world > 1 and dist.is_initialized():
        gathered = [None] * world
        dist.all_gather_object(gathered, times)
        times = max(gathered, key=len)
    if len(times) < warmup + steps:
        return {"impl": "reference", "unavailable": f"the reference logged {len(times)} iteration times, expected "
                f"{warmup + steps}"}
    timed = times[warmup:warmup + steps]
    ms = sum(timed) / len(timed)
    value = 512.0 / (ms / 1e3)
    max_mb = torch.cuda.max_memory_allocated() / 2 ** 20
    return {
        "impl": "reference",
        "metric": "samples/s (GPT-3 1.3B, GBS 512, searched plan)", "value": round(value, 3), "unit": "samples/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 2), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": round(value / PUBLISHED_SAMPLES_PER_S, 3), "dtype": dtype,
        "data": "synthetic (the reference's own get_batch: tokens created on the device, runtime/pretrain_gpt.py:50-62;"
                " random-init weights)",
        "config": {"model": "GPT-3 1.3B (24L, h2048, 16x128 heads, ffn 8192, seq 2048, vocab 51200, dropout 0.1)",
                   "global_batch": 512, "seq_len": 2048,
                   "parallelism": f"pp1-tp1-dp{world}-mbs{mbs}" + ("-recompute" if recompute else ""),
                   "num_microbatches": 512 // (mbs * world),
                   "timing": "the reference's own 'elapsed time per iteration' (host clock around an iteration whose "
                             "timers synchronise the device), as its per-rank CSV stores it",
                   "stand_ins": "apex FusedAdam / amp_C -> torch fused AdamW / _foreach kernels; torch._six",
                   "max_allocated_mb": round(max_mb), "iteration_ms": [round(t, 1) for t in times]},
        "e2e": {"value": round(value, 3), "unit": "samples/s", "ms_per_step": round(ms, 2),
                "note": "the reference's iteration already contains batch creation and the loss read-back"},
    }
