"""The resharding micro-benchmark's walk tp 4 -> 2 -> 1 -> 2 -> 4 on four gloo ranks: every intermediate shard is the
right slice of the global tensor, the round trip is exact, and one JSON line per transition comes out."""
import importlib.util
import json
import os

from dist_utils import run_ranks

BENCH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "reshard_bench.py")


def _worker(rank, world, out_path):
    import torch
    spec = importlib.util.spec_from_file_location("reshard_bench", BENCH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    lines = []
    ok = mod.run(tokens=64, hidden=32, iters=1, dtype=torch.float32, emit=lambda s, flush=True: lines.append(s))
    assert ok
    if rank == 0:
        with open(out_path, "w") as f:
            f.write("\n".join(lines))


def test_walk_down_and_up_is_exact_and_reports_every_transition(tmp_path):
    out = str(tmp_path / "lines.txt")
    run_ranks(_worker, 4, out)
    rows = [json.loads(l) for l in open(out).read().splitlines()]
    steps = [(r["from"], r["to"]) for r in rows if r.get("case") == "reshard"]
    assert steps == [("tp4-dp1", "tp2-dp2"), ("tp2-dp2", "tp1-dp4"), ("tp1-dp4", "tp2-dp2"), ("tp2-dp2", "tp4-dp1")]
    assert rows[-1] == {"round_trip_equal": True, "transitions": 4}
    for r in rows[:-1]:
        # a rank's shard is 1/4 of the tensor; the busiest rank receives half of its new shard or all of it
        assert r["bytes_received_per_rank"] in (1024, 2048) and r["timed_on"] == "host"
    assert rows[0]["bytes_received_per_rank"] == 2048      # tp 4 -> 2: ranks 2 and 3 hold nothing of their new shard
