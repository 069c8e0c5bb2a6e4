"""Failure detection on the host: per-rank heartbeats, a watchdog that notices a silent or dead rank between steps, and a step
deadline.  (The reference has no failure detection beyond the 20-minute process-group timeout, src/nanotron/distributed.py:18,
and relies on periodic checkpoints plus a manual relaunch.)

Everything here runs on the CPU and touches no GPU state, so a failed peer is reported *before* the next kernel or collective
is launched towards it; device-side waits are bounded separately (they give up and set a status word, see
``nanotron_b200.parallel.symm.CommTimeoutError``).  Recovery stays checkpoint-restart: survivors raise ``RankFailureError`` and
exit non-zero, the launcher restarts the job from ``latest.txt``.

A heartbeat is a small JSON file per rank in a directory every rank can see (node-local /dev/shm for one node, a shared file
system across nodes): ``{"rank", "step", "time", "pid", "state"}``, rewritten atomically by a daemon thread.
"""
from __future__ import annotations

import json
import os
import threading
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional


class RankFailureError(RuntimeError):
    """One or more peers stopped reporting (or reported a failure)."""

    def __init__(self, failed: Dict[int, str]):
        self.failed = failed
        super().__init__("rank failure detected: " + ", ".join(f"rank {r}: {why}" for r, why in sorted(failed.items())))


class StepDeadlineExceeded(RuntimeError):
    pass


@dataclass
class Beat:
    rank: int
    step: int
    time: float
    pid: int
    state: str  # "running" | "done" | "failed"


class Heartbeat:
    """Writes this rank's beat every ``interval`` seconds from a daemon thread; ``beat(step)`` records progress."""

    def __init__(self, directory: str, rank: int, interval: float = 1.0):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.rank, self.interval = rank, interval
        self._step = 0
        self._state = "running"
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._write()

    def path(self, rank: Optional[int] = None) -> Path:
        return self.dir / f"rank_{self.rank if rank is None else rank}.json"

    def _write(self):
        tmp = self.path().with_suffix(".tmp")
        with open(tmp, "w") as f:
            json.dump({"rank": self.rank, "step": self._step, "time": time.time(), "pid": os.getpid(), "state": self._state}, f)
        os.replace(tmp, self.path())  # atomic: readers never see a partial file

    def start(self) -> "Heartbeat":
        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self._write()
                except OSError:
                    pass  # a full or unreachable directory must not take the training process down

        self._thread = threading.Thread(target=loop, name="ntb-heartbeat", daemon=True)
        self._thread.start()
        return self

    def beat(self, step: int):
        self._step = step
        self._write()

    def stop(self, state: str = "done"):
        self._state = state
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
        try:
            self._write()
        except OSError:
            pass


class Watchdog:
    """Reads the peers' beats.  A peer is failed when it says so, when its beat is older than ``timeout`` seconds, or when it
    never appeared within ``startup_timeout``."""

    def __init__(self, directory: str, rank: int, world_size: int, timeout: float = 60.0, startup_timeout: Optional[float] = None):
        self.dir = Path(directory)
        self.rank, self.world_size, self.timeout = rank, world_size, timeout
        self.startup_timeout = startup_timeout if startup_timeout is not None else max(timeout, 120.0)
        self._t0 = time.time()

    def read(self, rank: int) -> Optional[Beat]:
        try:
            with open(self.dir / f"rank_{rank}.json") as f:
                return Beat(**json.load(f))
        except (OSError, ValueError, TypeError):
            return None

    def failed_ranks(self) -> Dict[int, str]:
        now = time.time()
        failed = {}
        for r in range(self.world_size):
            if r == self.rank:
                continue
            b = self.read(r)
            if b is None:
                if now - self._t0 > self.startup_timeout:
                    failed[r] = f"no heartbeat after {now - self._t0:.0f} s"
            elif b.state == "failed":
                failed[r] = f"reported failure at step {b.step}"
            elif b.state == "running" and now - b.time > self.timeout:
                failed[r] = f"last heartbeat {now - b.time:.1f} s ago at step {b.step}"
        return failed

    def raise_if_failed(self):
        failed = self.failed_ranks()
        if failed:
            raise RankFailureError(failed)

    def slowest(self) -> Optional[Beat]:
        beats = [b for b in (self.read(r) for r in range(self.world_size)) if b is not None]
        return min(beats, key=lambda b: b.step) if beats else None


class StepDeadline:
    """Wall-clock budget for one training step: ``with StepDeadline(seconds): step()`` raises after the fact when the step took
    longer (a hung collective is ended by the process-group timeout; this turns a merely slow step into a visible error)."""

    def __init__(self, seconds: Optional[float]):
        self.seconds = seconds

    def __enter__(self):
        self._t0 = time.time()
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is None and self.seconds is not None and time.time() - self._t0 > self.seconds:
            raise StepDeadlineExceeded(f"training step took {time.time() - self._t0:.1f} s, deadline {self.seconds:.1f} s")
        return False


def from_env(rank: int, world_size: int):
    """(Heartbeat, Watchdog) configured by NANOTRON_HEARTBEAT_DIR / NANOTRON_HEARTBEAT_INTERVAL / NANOTRON_HEARTBEAT_TIMEOUT, or
    (None, None) when no directory is set."""
    d = os.environ.get("NANOTRON_HEARTBEAT_DIR")
    if not d:
        return None, None
    interval = float(os.environ.get("NANOTRON_HEARTBEAT_INTERVAL", "1.0"))
    timeout = float(os.environ.get("NANOTRON_HEARTBEAT_TIMEOUT", "60.0"))
    return Heartbeat(d, rank, interval).start(), Watchdog(d, rank, world_size, timeout)
