"""Host-side failure detection between steps.

The reference has no watchdog of any kind (its only resilience is ``--resume_from_checkpoint``);
a rank that dies leaves the others blocked in their next collective until the job is killed.
Here every rank runs a small heartbeat thread against the job's key-value store:

* ``beat/<rank>``  wall-clock time of the rank's last heartbeat,
* ``fail/<rank>``  reason string written by ``report_failure`` (an exception handler calls it
                   before the rank leaves).

``check()`` is called between steps, before the next kernel or collective is launched. It raises
``PeerFailure`` when some rank reported an error or stopped beating for ``dead_after_s`` seconds,
so that the surviving ranks stop launching work, leave cleanly and the job can be restarted from
the last checkpoint. Nothing here touches a GPU: device-side waits have their own iteration
limits and report through the kernel status word (``ops._lib.read_status``).
"""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class HealthMonitor:
    def __init__(self, rank: int, world: int, store=None, heartbeat_s: float = 1.0,
                 dead_after_s: float = 30.0, prefix: str = "e2h_health"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = dist.PrefixStore(prefix, store)
        self.rank, self.world = rank, world
        self.heartbeat_s, self.dead_after_s = heartbeat_s, dead_after_s
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, float] = {}
        self._start_time = time.time()

    # ------------------------------------------------------------------ own liveness
    def _beat(self) -> None:
        self.store.set(f"beat/{self.rank}", repr(time.time()))

    def _loop(self) -> None:
        while not self._stop.wait(self.heartbeat_s):
            try:
                self._beat()
            except Exception:  # noqa: BLE001 -- the store went away with rank 0
                return

    def start(self) -> "HealthMonitor":
        self._beat()
        self._thread = threading.Thread(target=self._loop, name="e2h-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.heartbeat_s + 1.0)

    def report_failure(self, reason: str) -> None:
        self.store.set(f"fail/{self.rank}", reason[:500])

    # ------------------------------------------------------------------ peers
    def _get(self, key: str) -> Optional[str]:
        try:
            if not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:  # noqa: BLE001
            return None

    def peer_status(self) -> Dict[int, str]:
        """rank -> "ok" | "failed: <reason>" | "silent <seconds>s"."""
        now, out = time.time(), {}
        for r in range(self.world):
            if r == self.rank:
                out[r] = "ok"
                continue
            why = self._get(f"fail/{r}")
            if why is not None:
                out[r] = f"failed: {why}"
                continue
            beat = self._get(f"beat/{r}")
            last = float(beat) if beat is not None else self._start_time
            silent = now - last
            out[r] = "ok" if silent < self.dead_after_s else f"silent {silent:.1f}s"
        return out

    def check(self) -> None:
        for r, st in self.peer_status().items():
            if st != "ok":
                raise PeerFailure(r, st)


def guarded_step(monitor: Optional[HealthMonitor], fn, *args, **kwargs):
    """Run one training / generation step under the monitor: peers are checked first, and an
    exception raised by the step is published before it propagates."""
    if monitor is not None:
        monitor.check()
    try:
        return fn(*args, **kwargs)
    except Exception as e:  # noqa: BLE001
        if monitor is not None and not isinstance(e, PeerFailure):
            monitor.report_failure(f"{type(e).__name__}: {e}")
        raise
