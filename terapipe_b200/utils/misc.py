"""Host-side helpers: watchdog timeout, seeding, slice arithmetic, memory report.

Counterparts of the reference's utils.py (:11-111).
"""
from __future__ import annotations

import builtins
import errno
import functools
import gc
import os
import random
import signal
import threading
from typing import List

import numpy as np
import torch


class TimeoutError(Exception):  # noqa: A001 - name kept for callers of the reference API
    pass


def timeout(seconds: int = 10, error_message: str = os.strerror(errno.ETIME)):
    """Decorator: raise :class:`TimeoutError` in the main thread after ``seconds``.

    Uses SIGALRM, so it only arms in the main thread of the process; elsewhere the
    function runs unguarded (a per-rank :class:`terapipe_b200.utils.watchdog.Watchdog`
    covers worker threads)."""
    def decorator(func):
        @functools.wraps(func)
        def wrapper(*args, **kwargs):
            if threading.current_thread() is not threading.main_thread():
                return func(*args, **kwargs)

            def on_alarm(signum, frame):
                raise TimeoutError(error_message)

            previous = signal.signal(signal.SIGALRM, on_alarm)
            signal.alarm(int(seconds))
            try:
                return func(*args, **kwargs)
            finally:
                signal.alarm(0)
                signal.signal(signal.SIGALRM, previous)
        return wrapper
    return decorator


def suppress_output(rank: int) -> None:
    """Make ``print`` silent on every rank but 0 unless called with ``force=True``."""
    original = builtins.print

    def rank_print(*args, **kwargs):
        force = kwargs.pop("force", False)
        if force:
            original(f"rank #{rank}:", *args, **kwargs)
        elif rank == 0:
            original(*args, **kwargs)

    builtins.print = rank_print


def set_random_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)


def uniform_slice(length: int, n_slices: int) -> List[int]:
    """``n_slices`` lengths summing to ``length``; the first ``length % n_slices`` get one more."""
    base, extra = divmod(length, n_slices)
    return [base + (1 if i < extra else 0) for i in range(n_slices)]


def mem_report(printer=print) -> dict:
    """Total bytes of live tensor storages per device, found by walking the gc."""
    seen, totals = set(), {}
    for obj in gc.get_objects():
        try:
            if not torch.is_tensor(obj):
                continue
            storage = obj.untyped_storage()
        except Exception:
            continue
        key = storage.data_ptr()
        if key in seen or key == 0:
            continue
        seen.add(key)
        dev = str(obj.device)
        totals[dev] = totals.get(dev, 0) + storage.nbytes()
    for dev, nbytes in sorted(totals.items()):
        printer(f"{dev}: {nbytes / 2**20:.2f} MiB in {len(seen)} storages")
    return totals
