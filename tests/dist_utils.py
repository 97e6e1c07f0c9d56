"""Spawns gloo ranks on CPU for multi-process tests (rendezvous on 127.0.0.1)."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        torch.set_num_threads(1)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


_CTX = None


def _context():
    """Ranks are forked from a server process that has already imported torch (a fresh interpreter per rank spends
    seconds on that import); the server itself never initialises a process group or starts threads."""
    global _CTX
    if _CTX is None:
        _CTX = mp.get_context("forkserver")
        _CTX.set_forkserver_preload(["torch", "torch.distributed", "numpy", "superscaler_b200.runtime.trainer",
                                     "superscaler_b200.data.synthetic", "superscaler_b200.runtime.checkpointing"])
    return _CTX


def run_ranks(fn, world: int, *args, timeout: float = 240.0):
    ctx = _context()
    errq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    assert not alive, "ranks timed out"
    assert not errs, "\n".join(f"[rank {r}]\n{tb}" for r, tb in errs)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
