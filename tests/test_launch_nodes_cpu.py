"""The multi-node launcher, rehearsed on one machine: two "nodes" of one process each (local shells instead of ssh)
train a data-parallel plan together, and a node that fails takes the job down instead of leaving the other waiting."""
import glob
import json
import os
import socket
import subprocess
import sys

from helpers import tiny_gpt_plan

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(tmp_path, extra, iters=2):
    plan = tmp_path / "plan.json"
    plan.write_text(json.dumps(tiny_gpt_plan(num_gpus=(2,), tp=[1])))
    logs = str(tmp_path / "logs")
    cmd = [sys.executable, os.path.join(ROOT, "examples", "launch_nodes.py"), "--hosts", "a,b", "--ssh", "local", "--plan",
           str(plan), "--log-dir", logs, "--gpus-per-node", "1", "--master-port", str(_port()), "--train-iters", str(iters),
           "--", "--hidden-dropout", "0", "--attention-dropout", "0"] + extra
    return subprocess.run(cmd, capture_output=True, text=True, timeout=300), logs


def test_two_nodes_train_one_data_parallel_plan(tmp_path):
    r, logs = _launch(tmp_path, [])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    node_logs = sorted(glob.glob(os.path.join(logs, "launcher_node*.log")))
    assert len(node_logs) == 2
    text = open(node_logs[0]).read() + open(node_logs[1]).read()
    assert "iteration        2/       2" in text
    assert len(glob.glob(os.path.join(logs, "csv", "*.csv"))) == 2          # one per rank


def test_a_failing_node_ends_the_job(tmp_path):
    r, logs = _launch(tmp_path, ["--health-check", "--inject-failure", "1:2"], iters=4)
    assert r.returncode != 0
    assert "stopping the other nodes" in r.stdout
