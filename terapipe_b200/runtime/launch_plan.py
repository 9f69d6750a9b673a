"""Recorded launch plans: replay the kernel launches of a step segment without re-deriving
their arguments.

A pipeline stage that talks to its neighbours through NCCL cannot be captured in one CUDA graph,
so its kernels are launched from Python, a dozen per layer and token slice.  Every argument of
those launches is static (buffers are allocated once, slices are row ranges), yet computing them
again each step (pointer arithmetic, dictionary look-ups, argument marshalling) costs more host
time per launch than a small kernel runs on the device.  ``RecordingLibrary`` wraps the ctypes
kernel library: while a segment is being recorded, every call made through the wrapper is
executed and also appended to the segment as ``(function, arguments)``; afterwards
``SegmentCache.run`` replays the list.  Communication stays outside the segments.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Hashable, List, Optional, Tuple

Segment = List[Tuple[Callable[..., Any], tuple]]


class RecordingLibrary:
    """Attribute access returns the wrapped library's functions; calls are recorded while a
    segment is open.  Non-zero return codes abort the recording (the segment is dropped)."""

    def __init__(self, lib):
        object.__setattr__(self, "_lib", lib)
        object.__setattr__(self, "_segment", None)
        object.__setattr__(self, "_failed", False)

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not callable(fn):
            return fn

        def call(*args):
            rc = fn(*args)
            if self._segment is not None:
                if isinstance(rc, int) and rc != 0:
                    object.__setattr__(self, "_failed", True)
                self._segment.append((fn, args))
            return rc

        object.__setattr__(self, name, call)   # next access skips __getattr__
        return call

    def begin(self) -> None:
        if self._segment is not None:
            raise RuntimeError("a segment is already being recorded")
        object.__setattr__(self, "_segment", [])
        object.__setattr__(self, "_failed", False)

    def end(self) -> Optional[Segment]:
        seg, failed = self._segment, self._failed
        object.__setattr__(self, "_segment", None)
        return None if failed else seg


class SegmentCache:
    """``run(key, fn, *args)``: the first time, call ``fn(*args)`` while recording the library
    calls it makes; later, replay them.  ``token`` guards the recordings: when it changes (for
    example the launch stream), everything is recorded afresh."""

    def __init__(self, lib: RecordingLibrary, on_error: Optional[Callable[[int, str], None]] = None):
        self.lib = lib
        self.on_error = on_error
        self.segments: Dict[Hashable, Segment] = {}
        self.token: Any = None
        self.replayed = 0

    def validate(self, token) -> None:
        if token != self.token:
            self.segments.clear()
            self.token = token

    def run(self, key: Hashable, fn: Callable[..., Any], *args) -> None:
        seg = self.segments.get(key)
        if seg is None:
            self.lib.begin()
            try:
                fn(*args)
            finally:
                seg = self.lib.end()
            if seg is not None:
                self.segments[key] = seg
            else:
                # a dropped recording would leave the others with call counters that no longer
                # line up with what the host derives: start over
                self.segments.clear()
            return
        for f, a in seg:
            rc = f(*a)
            if rc and self.on_error is not None:
                self.on_error(rc, getattr(f, "__name__", "kernel"))
        self.replayed += len(seg)
