"""Lightweight tracing: NVTX ranges and a per-slice device timeline.

``nvtx_range`` marks (slice, layer, phase) regions for Nsight; it is a no-op without CUDA.
``SliceTimeline`` brackets the receive / compute / send of every token slice with CUDA events
and writes ``[{"pass", "batch_slice", "token_slice", "stage", "t_start_ms", "t_end_ms"}, ...]``
as JSON, which shows the pipeline's fill, steady state and bubbles per stage.
"""
from __future__ import annotations

import contextlib
import json
from typing import List

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class SliceTimeline:
    def __init__(self, stage: int, enabled: bool = True):
        self.stage, self.enabled = stage, enabled and torch.cuda.is_available()
        self._open = []
        self._origin = None

    def begin_iteration(self):
        if self.enabled:
            self._open = []
            self._origin = torch.cuda.Event(enable_timing=True)
            self._origin.record()

    @contextlib.contextmanager
    def slice(self, which: str, batch_slice: int, token_slice: int):
        if not self.enabled:
            yield
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        with nvtx_range(f"{which} b{batch_slice} s{token_slice}"):
            yield
        e1.record()
        self._open.append((which, batch_slice, token_slice, e0, e1))

    def records(self) -> List[dict]:
        if not self.enabled or self._origin is None:
            return []
        torch.cuda.synchronize()
        return [{"pass": w, "batch_slice": b, "token_slice": s, "stage": self.stage,
                 "t_start_ms": self._origin.elapsed_time(e0), "t_end_ms": self._origin.elapsed_time(e1)}
                for w, b, s, e0, e1 in self._open]

    def dump(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.records(), f)
