"""The benchmark entry point's contract that can be checked without a GPU: the reference arm answers with one JSON
line and exit code 0, and the committed plans `bench.py --gpus N` trains are consistent with the benchmark."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_unavailable_and_exits_zero():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                        "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and isinstance(out["unavailable"], str) and "\n" not in out["unavailable"]


@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_committed_bench_plans(n):
    from superscaler_b200.runtime.trainer import _validate_plan
    with open(os.path.join(ROOT, "plans", f"gpt_1_3B_{n}gpu_b200.json")) as f:
        plan = json.load(f)
    _validate_plan(plan)
    assert sum(plan["num_gpus"]) == n and plan["global_batch_size"] == 512
    assert plan["global_batch_size"] % plan["micro_batch_size"] == 0
    assert (plan["num_layers"], plan["hidden_size"], plan["num_attention_heads"], plan["kv_channels"],
            plan["seq_length"], plan["vocab_size"]) == (24, 2048, 16, 128, 2048, 51200)


@pytest.mark.parametrize("model,name,gbs", [("t5", "t5_770M", 512), ("resnet", "resnet_1B", 768)])
@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_committed_plans_of_the_other_two_benchmark_models(model, name, gbs, n):
    """`bench.py --model t5|resnet --gpus N` trains these files: right model, GPU count and global batch, and the
    per-GPU micro-batch is one the database has a table for."""
    from superscaler_b200.runtime.trainer import _validate_plan
    with open(os.path.join(ROOT, "plans", f"{name}_{n}gpu_b200.json")) as f:
        plan = json.load(f)
    _validate_plan(plan)
    assert plan["model_name"] == model and sum(plan["num_gpus"]) == n and plan["global_batch_size"] == gbs
    assert gbs % plan["micro_batch_size"] == 0
    per_gpu = plan["micro_batch_size"] // plan["data_parallel_size_of_each_op"][0][0]
    table = os.path.join(ROOT, "profiled-time-b200", f"{name}_mbs{per_gpu}_tp1_algo0.csv")
    assert os.path.isfile(table), table
    if model == "t5":
        assert plan["relative_position_bias"] is True and plan["activation"] == "relu"
