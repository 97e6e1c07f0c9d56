"""Host-side failure detection for multi-rank runs.

The reference has none: a rank that dies leaves the others blocked in a collective until somebody kills the job
(runtime/scripts/run_gpt_2nodes.sh:55-62 sweeps the nodes with `kill -9`).  Here every rank publishes a heartbeat
and, when it fails, the reason, in a key-value store every rank can reach (the TCPStore of the rendezvous or any
object with `set` / `get` / `check`); ranks look at it between steps, BEFORE they launch the next collective, so a
failure turns into a `PeerFailure` exception on the survivors instead of a hang.

    monitor = HealthMonitor(store, rank, world, stale_after_s=60)
    for batch in data:
        monitor.beat(step)                 # publish, then raise PeerFailure if a peer failed or went silent
        with monitor.guard():              # publishes this rank's own exception before re-raising it
            trainer.train_step(batch)

The device side has the matching property: every kernel that waits on another GPU gives up after a bounded time and
reports `kStatusPeerTimeout` in the status word (`ops/native.py::check_status`), see csrc/comm_sm100.cu.  The trainer
reads that word wherever the host synchronises anyway (`Trainer.loss_value`, `save_checkpoint`) and raises
`DeviceStatusError`, publishing the failure through the attached monitor (`trainer.health_monitor`).
"""
from __future__ import annotations

import contextlib
import time
from typing import Dict, Optional


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class DeviceStatusError(RuntimeError):
    """A kernel of this rank returned from a bounded wait without its data (status word != 0)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"device status {code}: {message}")
        self.code = code


class DictStore:
    """In-process stand-in for a distributed store (tests, single-process runs)."""

    def __init__(self):
        self.d: Dict[str, bytes] = {}

    def set(self, k: str, v) -> None:
        self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        return self.d[k]

    def check(self, keys) -> bool:
        return all(k in self.d for k in keys)


class HealthMonitor:
    def __init__(self, store, rank: int, world: int, stale_after_s: float = 120.0, prefix: str = "health",
                 clock=time.time):
        self.store, self.rank, self.world = store, rank, world
        self.stale_after_s, self.prefix, self.clock = stale_after_s, prefix, clock
        self._last_seen: Dict[int, tuple] = {}

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def _get(self, key: str) -> Optional[str]:
        if not self.store.check([key]):
            return None
        return self.store.get(key).decode()

    def publish_failure(self, reason: str) -> None:
        self.store.set(self._key("failed", self.rank), reason[:2000])

    def beat(self, step: int, check: bool = True) -> None:
        """Publishes (step, time) for this rank; with check=True raises PeerFailure for a failed or silent peer."""
        self.store.set(self._key("hb", self.rank), f"{step}:{self.clock():.3f}")
        if check:
            self.check_peers()

    def check_peers(self) -> None:
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            failed = self._get(self._key("failed", r))
            if failed is not None:
                raise PeerFailure(r, failed)
            hb = self._get(self._key("hb", r))
            if hb is None:
                first = self._last_seen.setdefault(r, (None, now))[1]
                if now - first > self.stale_after_s:
                    raise PeerFailure(r, f"never published a heartbeat within {self.stale_after_s:.0f} s")
                continue
            prev = self._last_seen.get(r)
            if prev is None or prev[0] != hb:
                self._last_seen[r] = (hb, now)       # progress observed on OUR clock: no cross-host clock needed
            elif now - prev[1] > self.stale_after_s:
                raise PeerFailure(r, f"heartbeat stuck at step {hb.split(':')[0]} for {now - prev[1]:.0f} s")

    @contextlib.contextmanager
    def guard(self):
        try:
            yield
        except PeerFailure:
            raise
        except BaseException as e:  # noqa: BLE001 - the reason travels to the peers, the exception goes on
            try:
                self.publish_failure(f"{type(e).__name__}: {e}")
            finally:
                raise


def store_from_env(rank: int, world: int, port_offset: int = 7, timeout_s: float = 60.0):
    """A TCPStore of its own for the heartbeats, on MASTER_ADDR : MASTER_PORT + port_offset (rank 0 hosts it), so
    that the monitor does not share a connection with the process group it watches over."""
    import datetime
    import os

    import torch.distributed as dist
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + port_offset
    return dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=timeout_s),
                         wait_for_workers=False)


def device_status_message(code: int) -> str:
    return {0: "ok", 1: "a kernel gave up waiting on one of its own barriers (mbarrier time limit)",
            2: "a kernel gave up waiting for a peer GPU (peer time limit): a rank is late or gone"}.get(
        code, f"unknown status {code}")
