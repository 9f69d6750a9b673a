"""Host-side liveness: a per-rank watchdog thread and heartbeat files the launcher can watch.

The reference guards a run with a SIGALRM timeout only (utils.py:14-30).  Here every rank may
start a :class:`Watchdog` that (a) touches ``<dir>/rank<k>.hb`` whenever the training loop calls
``beat()`` and (b) calls ``on_timeout`` (default: dump stacks and exit the process with code
70) when no beat arrived for ``timeout_s``.  :func:`stale_ranks` lets a launcher or a test find
ranks whose heartbeat file is older than a limit.  Nothing here touches the GPU.
"""
from __future__ import annotations

import faulthandler
import os
import sys
import threading
import time
from typing import Callable, List, Optional


class Watchdog:
    def __init__(self, timeout_s: float, rank: int = 0, heartbeat_dir: Optional[str] = None,
                 on_timeout: Optional[Callable[[], None]] = None, poll_s: float = 0.2):
        self.timeout_s, self.rank, self.poll_s = timeout_s, rank, poll_s
        self.heartbeat_dir = heartbeat_dir
        self.on_timeout = on_timeout or self._default_timeout
        self._last = time.monotonic()
        self._stop = threading.Event()
        self.fired = False
        self._thread = threading.Thread(target=self._run, name=f"watchdog-{rank}", daemon=True)
        if heartbeat_dir:
            os.makedirs(heartbeat_dir, exist_ok=True)

    def _default_timeout(self):
        sys.stderr.write(f"[watchdog] rank {self.rank}: no progress for {self.timeout_s}s\n")
        faulthandler.dump_traceback(file=sys.stderr)
        os._exit(70)

    def start(self) -> "Watchdog":
        self.beat()
        self._thread.start()
        return self

    def beat(self) -> None:
        self._last = time.monotonic()
        if self.heartbeat_dir:
            path = os.path.join(self.heartbeat_dir, f"rank{self.rank}.hb")
            with open(path, "w") as f:
                f.write(str(time.time()))

    def stop(self) -> None:
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=2 * self.poll_s + 1)

    def _run(self):
        while not self._stop.wait(self.poll_s):
            if time.monotonic() - self._last > self.timeout_s:
                self.fired = True
                self.on_timeout()
                return

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
        return False


def stale_ranks(heartbeat_dir: str, world_size: int, max_age_s: float) -> List[int]:
    """Ranks whose heartbeat file is missing or older than ``max_age_s``."""
    now, out = time.time(), []
    for r in range(world_size):
        path = os.path.join(heartbeat_dir, f"rank{r}.hb")
        try:
            if now - os.path.getmtime(path) > max_age_s:
                out.append(r)
        except OSError:
            out.append(r)
    return out
