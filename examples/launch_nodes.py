"""Starts one training job on several nodes: `examples/run_node.sh` once per host, over ssh, with NNODES / NODE_RANK /
MASTER_ADDR filled in, and ends the whole job as soon as one node fails (a rank that ran out of memory or lost a
peer otherwise leaves the others waiting in a collective).

    python examples/launch_nodes.py --hosts node0,node1 --plan plans/gpt_13B_16gpu.json --log-dir logs/ \\
        [--gpus-per-node 8] [--master-port 7000] [--workdir /path/to/repo] [--train-iters 3] [-- extra pretrain flags]

The first host is the rendezvous master.  `--ssh` is the remote-shell command (default `ssh -o BatchMode=yes`);
`--ssh local` runs every "node" as a local process instead, which is how a multi-node launch is rehearsed on one
machine (give each node one process with --gpus-per-node 1).  Reference counterpart: the parallel-ssh launch and the
kill-on-failure loop of runtime/scripts/run_gpt_2nodes.sh:55-62.
"""
from __future__ import annotations

import argparse
import os
import shlex
import signal
import subprocess
import sys
import time
from typing import List


def node_command(a, rank: int, n: int, master: str, extra: List[str]) -> str:
    env = (f"NNODES={n} NODE_RANK={rank} GPUS_PER_NODE={a.gpus_per_node} MASTER_ADDR={master} "
           f"MASTER_PORT={a.master_port} TRAIN_ITERS={a.train_iters}")
    args = " ".join(shlex.quote(x) for x in [a.plan, a.log_dir] + extra)
    return f"cd {shlex.quote(a.workdir)} && {env} bash examples/run_node.sh {args}"


def launch(a, extra: List[str]) -> int:
    hosts = [h for h in (a.hosts.split(",") if a.hosts else open(a.hostfile).read().split()) if h]
    assert hosts, "no hosts given"
    master = a.master_addr or ("127.0.0.1" if a.ssh == "local" else hosts[0])
    procs = []
    for rank, host in enumerate(hosts):
        cmd = node_command(a, rank, len(hosts), master, extra)
        argv = ["bash", "-c", cmd] if a.ssh == "local" else shlex.split(a.ssh) + [host, cmd]
        out = open(os.path.join(a.log_dir, f"launcher_node{rank}.log"), "w")
        procs.append((host, subprocess.Popen(argv, stdout=out, stderr=subprocess.STDOUT, start_new_session=True), out))
        print(f"[launch_nodes] node {rank} on {host}: pid {procs[-1][1].pid}", flush=True)
    code = 0
    try:
        while True:
            states = [p.poll() for _, p, _ in procs]
            failed = [(h, s) for (h, _, _), s in zip(procs, states) if s not in (None, 0)]
            if failed:
                code = failed[0][1]
                print(f"[launch_nodes] node on {failed[0][0]} left with code {code}: stopping the other nodes", flush=True)
                break
            if all(s == 0 for s in states):
                break
            time.sleep(0.5)
    finally:
        for _, p, out in procs:
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)       # the session this launcher started, nothing else
                except ProcessLookupError:
                    pass
        deadline = time.time() + 20
        for _, p, out in procs:
            try:
                p.wait(timeout=max(0.1, deadline - time.time()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
            out.close()
    return code


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    extra: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, extra = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--hosts", default=None, help="comma-separated host names, the master first")
    ap.add_argument("--hostfile", default=None, help="file with one host per line (instead of --hosts)")
    ap.add_argument("--plan", required=True)
    ap.add_argument("--log-dir", required=True)
    ap.add_argument("--gpus-per-node", type=int, default=8)
    ap.add_argument("--master-addr", default=None)
    ap.add_argument("--master-port", type=int, default=7000)
    ap.add_argument("--train-iters", type=int, default=3)
    ap.add_argument("--workdir", default=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ap.add_argument("--ssh", default="ssh -o BatchMode=yes")
    a = ap.parse_args(argv)
    assert a.hosts or a.hostfile, "give --hosts or --hostfile"
    os.makedirs(a.log_dir, exist_ok=True)
    return launch(a, extra)


if __name__ == "__main__":
    sys.exit(main())
