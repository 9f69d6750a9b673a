"""Per-stage latency model and the slice-schedule dynamic program.

Pipeline of the reference's planner (latency_model.py:16-193), re-implemented:

1. A *latency table* maps ``(batch, slice_len, context_len)`` to measured forward, backward
   and optimizer times of ONE layer (keys ``"b_s_c"``; written by the latency measurer).
2. ``fit_single_layer_model`` turns it into a dense grid ``t[b, s/gap, c/gap]``:
   context-free time ``t0[b, s]`` (measured where available, otherwise a least-squares
   surface) plus a linear model of the context cost on features ``[b*s, b*c, b*s*c]``,
   times the layers per stage, plus two inter-stage transfers interpolated from the
   point-to-point table.
3. ``planning`` (C++, ``ops/csrc/host/planner.cpp``) minimises the sum of slice latencies
   under a cap ``t_max`` on any one slice; ``analysis_model`` scans ``t_max`` over the
   distinct grid values and keeps the schedule minimising
   ``sum_i t_i + (K-1) * max_i t_i + optimizer time``.

``step_gap`` (token granularity of the grid) is a parameter; the reference hard-codes 8.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..models.config import BATCH_CONFIGS, MODEL_CONFIGS

SCAN_GRID = (16, 16, 4)
STEP_GAP = 8

Scheme = List[Tuple[int, List[int]]]


def parse_json(raw: Dict[str, dict]) -> Dict[Tuple[int, int, int], dict]:
    return {tuple(int(v) for v in k.split("_")): val for k, val in raw.items()}


class SingleLayerLatency:
    """Dense latency grid of one pipeline stage, indexed ``[batch, slice/gap, context/gap]``."""

    def __init__(self, no_context, update_time, context_coef, comm_time, layers_per_stage,
                 step_gap=STEP_GAP):
        self.no_content_performance = np.asarray(no_context, dtype=np.float64)
        self.update_time = float(update_time)
        self.context_coef = np.asarray(context_coef, dtype=np.float64)  # w0, w_bs, w_bc, w_bsc
        self.comm_time = np.asarray(comm_time, dtype=np.float64)
        self.step_gap = step_gap
        nb, ns = self.no_content_performance.shape
        b = np.arange(nb, dtype=np.float64)[:, None, None]
        s = (np.arange(ns, dtype=np.float64) * step_gap)[None, :, None]
        c = (np.arange(ns, dtype=np.float64) * step_gap)[None, None, :]
        w0, w1, w2, w3 = self.context_coef
        ctx = w0 + w1 * b * s + w2 * b * c + w3 * b * s * c
        base = self.no_content_performance * layers_per_stage + 2.0 * self.comm_time
        self.latency_grid = np.ascontiguousarray(base[:, :, None] + ctx * layers_per_stage)

    def predict(self, batch_size, seqlen, context_len):
        g = self.step_gap
        assert seqlen % g == 0 and context_len % g == 0
        return self.latency_grid[batch_size, seqlen // g, context_len // g]


def _fit_context_model(rows, targets, holdout=0.25, seed=42):
    """Least squares of ``t(b,s,c) - t0(b,s)`` on ``[1, b*s, b*c, b*s*c]``; returns
    (coefficients, R^2 on a held-out quarter)."""
    X = np.asarray(rows, dtype=np.float64)
    y = np.asarray(targets, dtype=np.float64)
    if len(y) == 0:
        return np.zeros(4), float("nan")
    A = np.concatenate([np.ones((len(X), 1)), X], axis=1)
    idx = np.random.RandomState(seed).permutation(len(y))
    n_test = int(len(y) * holdout) if len(y) >= 8 else 0
    test, train = idx[:n_test], idx[n_test:]
    coef, *_ = np.linalg.lstsq(A[train], y[train], rcond=None)
    if (coef[1:] < 0).any():
        # More context can only cost time (the attention core reads more keys).  On a B200 the
        # context term of a slice is small against run-to-run noise, and an unconstrained fit
        # then returns negative slopes that make long contexts look cheap: fit with
        # non-negative coefficients instead.
        try:
            from scipy.optimize import nnls
            coef, _ = nnls(A[train], np.maximum(y[train], 0.0))
        except Exception:  # noqa: BLE001 - no scipy: clip
            coef = np.maximum(coef, 0.0)
    if n_test:
        resid = y[test] - A[test] @ coef
        denom = ((y[test] - y[test].mean()) ** 2).sum()
        r2 = 1.0 - (resid ** 2).sum() / denom if denom > 0 else float("nan")
    else:
        r2 = float("nan")
    return coef, r2


def fit_latency_tables(latency_table: Dict[Tuple[int, int, int], dict],
                       comm_table: Optional[dict], batch_size: int, seqlen: int,
                       layers_per_stage: int, step_gap: int = STEP_GAP,
                       fill_missing: bool = True, verbose: bool = False,
                       total_batch: Optional[int] = None) -> SingleLayerLatency:
    update_time = float(np.mean([t["update_mean"] for t in latency_table.values()]))
    wg = [t["wgrad_per_token_mean"] for t in latency_table.values() if "wgrad_per_token_mean" in t]
    if wg:
        # per-layer constant of an iteration: optimizer + whole-sequence weight gradients
        # per-token cost at the largest measured row count (small row counts under-use the GPU)
        rows = [k[0] * (k[1] + k[2]) for k, t in latency_table.items() if "wgrad_per_token_mean" in t]
        update_time += float(wg[int(np.argmax(rows))]) * seqlen * (total_batch or batch_size)
    ns = seqlen // step_gap + 1
    t0 = np.full((batch_size + 1, ns), np.inf)
    for (b, s, c), t in latency_table.items():
        if c == 0 and b <= batch_size and s % step_gap == 0 and s // step_gap < ns:
            t0[b, s // step_gap] = t["forward_mean"] + t["backward_mean"]
    if fill_missing:
        # a coarse measurement grid leaves holes: fill them with a least-squares surface
        # t0 ~ a + b1*b + b2*s + b3*b*s + b4*b*s^2 fitted on the measured points
        known = np.argwhere(np.isfinite(t0))
        if len(known) >= 5:
            bb, ss = known[:, 0].astype(float), known[:, 1].astype(float) * step_gap
            A = np.stack([np.ones_like(bb), bb, ss, bb * ss, bb * ss * ss], axis=1)
            coef, *_ = np.linalg.lstsq(A, t0[known[:, 0], known[:, 1]], rcond=None)
            gb, gs = np.meshgrid(np.arange(batch_size + 1, dtype=float),
                                 np.arange(ns, dtype=float) * step_gap, indexing="ij")
            surf = coef[0] + coef[1] * gb + coef[2] * gs + coef[3] * gb * gs + coef[4] * gb * gs * gs
            floor = float(np.min(t0[np.isfinite(t0)])) * 0.5
            surf = np.maximum(surf, floor)
            hole = ~np.isfinite(t0)
            hole[0, :] = False
            hole[:, 0] = False
            # batch sizes without any measurement stay infeasible: the surface is not trusted
            # outside the measured range (it made unmeasured small batches look free)
            for b in range(t0.shape[0]):
                if np.isfinite(t0[b]).sum() < 2:
                    hole[b, :] = False
            t0[hole] = surf[hole]
    rows, targets = [], []
    for (b, s, c), t in latency_table.items():
        if c > 0 and b <= batch_size and s % step_gap == 0 and s // step_gap < ns:
            base = t0[b, s // step_gap]
            val = t["forward_mean"] + t["backward_mean"] - base
            if np.isfinite(val):
                rows.append([b * s, b * c, b * s * c])
                targets.append(val)
    coef, r2 = _fit_context_model(rows, targets)
    if verbose:
        print("Linear regression score:", r2)
    comm = np.zeros((batch_size + 1, ns))
    if comm_table is not None:
        xp = np.asarray(comm_table["tensor_sizes"], dtype=np.float64)
        yp = np.asarray(comm_table["mean"], dtype=np.float64)
        tokens = np.arange(batch_size + 1)[:, None] * (np.arange(ns)[None, :] * step_gap)
        comm = np.interp(tokens, xp, yp)
        comm[0, :] = 0.0
        comm[:, 0] = 0.0
    model = SingleLayerLatency(t0, update_time, coef, comm, layers_per_stage, step_gap)
    model.r2 = r2
    return model


def fit_single_layer_model(model_name, model_parallel_size, layers_per_node,
                           data_dir="performance_model_data", step_gap=STEP_GAP,
                           batch_size=None, verbose=True, total_batch=None):
    """Load ``latency_model.<model>.mp_<mp>.json`` and ``<model>.communication_latency.json``
    from ``data_dir`` and fit the stage model."""
    with open(os.path.join(data_dir, f"latency_model.{model_name}.mp_{model_parallel_size}.json")) as f:
        table = parse_json(json.load(f))
    comm_path = os.path.join(data_dir, f"{model_name}.communication_latency.json")
    comm = json.load(open(comm_path)) if os.path.exists(comm_path) else None
    seqlen = MODEL_CONFIGS[model_name][2]
    if batch_size is None:
        batch_size = BATCH_CONFIGS.get(model_name, max(k[0] for k in table))
    batch_size = min(batch_size, max(k[0] for k in table))
    return fit_latency_tables(table, comm, batch_size, seqlen, layers_per_node, step_gap,
                              verbose=verbose, total_batch=total_batch)


# ------------------------------------------------------------------------- dynamic program
def _planning_numpy(grid, B, n, max_latency):
    """Reference implementation of the recurrences in NumPy (used when the host library is
    unavailable and as a cross-check in tests)."""
    gb, gs, gc = grid.shape
    inf = np.inf
    f = np.zeros((B + 1, n + 1))
    fmax = np.zeros((B + 1, n + 1))
    fstep = np.zeros((B + 1, n + 1), dtype=np.int64)
    for bs in range(1, B + 1):
        for acc in range(1, n + 1):
            best, best_s, best_max = inf, 0, 0.0
            if bs < gb:
                for s in range(1, acc + 1):
                    c = acc - s
                    if s >= gs or c >= gc:
                        continue
                    lat = grid[bs, s, c]
                    if not lat <= max_latency:
                        continue
                    tot = f[bs, c] + lat
                    if tot < best:
                        best, best_s, best_max = tot, s, max(fmax[bs, c], lat)
            f[bs, acc], fstep[bs, acc], fmax[bs, acc] = best, best_s, best_max
    g = np.zeros(B + 1)
    gmax = np.zeros(B + 1)
    gstep = np.zeros(B + 1, dtype=np.int64)
    for acc in range(1, B + 1):
        best, best_bs, best_max = inf, 0, 0.0
        for bs in range(1, acc + 1):
            tot = g[acc - bs] + f[bs, n]
            if tot < best:
                best, best_bs, best_max = tot, bs, max(gmax[acc - bs], fmax[bs, n])
        g[acc], gstep[acc], gmax[acc] = best, best_bs, best_max
    return g[B], gmax[B], fstep, gstep


def _dp_tables(grid, B, n, max_latency, use_native=True):
    """(sum, max, f_step, g_step) of the recurrences, from the C++ library when available."""
    lib = None
    if use_native:
        try:
            from ..ops.lib import host_lib
            lib = host_lib()
        except Exception:
            lib = None
    if lib is None:
        return _planning_numpy(grid, B, n, max_latency)
    fstep = np.zeros((B + 1, n + 1), dtype=np.int64)
    gstep = np.zeros(B + 1, dtype=np.int64)
    mx = ctypes.c_double(0.0)
    total = lib.tp_plan_slices(grid.ctypes.data, grid.shape[0], grid.shape[1], grid.shape[2],
                               B, n, float(max_latency), fstep.ctypes.data, gstep.ctypes.data,
                               ctypes.byref(mx))
    return total, mx.value, fstep, gstep


def _token_slices(fstep, bs, n, step_gap):
    """Backtrack one batch-slice size: token slices, last first, or None if infeasible."""
    lens, cur = [], n
    while cur > 0:
        s = int(fstep[bs, cur])
        if s <= 0:
            return None
        lens.append(s * step_gap)
        cur -= s
    return lens


def planning(latency_grid, total_batch_size, total_seqlen, pipelinelen, max_latency,
             step_gap=STEP_GAP, use_native=True, uniform_batch=False):
    """Best schedule whose every slice takes at most ``max_latency``.

    Returns ``(total_time, scheme)`` where ``total_time = (K-1) * max_slice + sum`` and
    ``scheme = [(batch_slice_size, [token slices, last first]), ...]`` (the same order the
    reference returns, latency_model.py:137-148), or ``(inf, None)``.

    ``uniform_batch=True`` only considers equal batch slices (sizes dividing the batch), so that
    every batch slice uses the same token slicing, which the runtimes require (the reference
    asserts it after planning, latency_model.py:240)."""
    assert total_seqlen % step_gap == 0
    grid = np.ascontiguousarray(latency_grid, dtype=np.float64)
    n = total_seqlen // step_gap
    B = int(total_batch_size)
    total, mx, fstep, gstep = _dp_tables(grid, B, n, max_latency, use_native)
    if uniform_batch:
        best = (float("inf"), None)
        for bs in range(1, B + 1):
            if B % bs or bs >= grid.shape[0]:
                continue
            lens = _token_slices(fstep, bs, n, step_gap)
            if lens is None:
                continue
            ctx, tot, big = 0, 0.0, 0.0
            for t in reversed(lens):
                lat = grid[bs, t // step_gap, ctx // step_gap]
                tot, big, ctx = tot + lat, max(big, lat), ctx + t
            cand = (B // bs) * tot + (pipelinelen - 1) * big
            if cand < best[0]:
                best = (cand, [(bs, list(lens)) for _ in range(B // bs)])
        return best
    if not np.isfinite(total):
        return float("inf"), None
    scheme: Scheme = []
    cur_b = B
    while cur_b > 0:
        bs = int(gstep[cur_b])
        scheme.append((bs, _token_slices(fstep, bs, n, step_gap)))
        cur_b -= bs
    return (pipelinelen - 1) * mx + total, scheme


def evaluate_split(latency_model: SingleLayerLatency, split_scheme: Scheme, pipelinelen,
                   layers_per_node):
    """Predicted iteration latency of a given schedule (token slices in chronological order)."""
    total, largest = 0.0, 0.0
    for batch_size, seq_splits in split_scheme:
        ctx = 0
        for seq_len in seq_splits:
            t = latency_model.predict(batch_size, seq_len, ctx)
            total += t
            largest = max(largest, t)
            ctx += seq_len
    return total + (pipelinelen - 1) * largest + latency_model.update_time * layers_per_node


def search_schedule(latency_model: SingleLayerLatency, total_batch_size, seqlen, pipelinelen,
                    layers_per_node, gap=1e-5, max_candidates: Optional[int] = None, progress=None,
                    uniform_batch=True):
    """Scan the slice-latency cap over the distinct grid values (ascending) and keep the
    best schedule; stops when ``cap * K`` alone exceeds the best total found."""
    grid = latency_model.latency_grid
    finite = grid[np.isfinite(grid)]
    candidates = np.unique(finite)
    if max_candidates and len(candidates) > max_candidates:
        candidates = candidates[np.linspace(0, len(candidates) - 1, max_candidates).astype(int)]
    best_latency, best_scheme, last = float("inf"), None, 0.0
    it = progress(candidates) if progress else candidates
    for cap in it:
        if cap * pipelinelen > best_latency:
            break
        if cap - last < gap:
            continue
        last = cap
        latency, scheme = planning(grid, total_batch_size, seqlen, pipelinelen, cap,
                                   latency_model.step_gap, uniform_batch=uniform_batch)
        if scheme is None:
            continue
        latency += layers_per_node * latency_model.update_time
        if latency < best_latency:
            best_latency = latency
            best_scheme = [(b, list(reversed(s))) for b, s in scheme]
    return best_scheme, best_latency


def analysis_model(model_name, total_batch_size, model_parallel_size, pipelinelen,
                   data_dir="performance_model_data", step_gap=STEP_GAP, n_layers=None,
                   verbose=True):
    """(scheme, latency) for a model/batch/TP/PP setting from the tables in ``data_dir``."""
    layers, _, seqlen, _ = MODEL_CONFIGS[model_name]
    layers = n_layers if n_layers is not None else layers
    layers_per_node = layers // pipelinelen
    lm = fit_single_layer_model(model_name, model_parallel_size, layers_per_node, data_dir,
                                step_gap, batch_size=max(total_batch_size,
                                                         BATCH_CONFIGS.get(model_name, 0)),
                                verbose=verbose, total_batch=total_batch_size)
    scheme, latency = search_schedule(lm, total_batch_size, seqlen, pipelinelen, layers_per_node)
    if verbose and scheme is not None:
        print(latency, scheme, len(scheme), evaluate_split(lm, scheme, pipelinelen, layers_per_node))
    return scheme, latency


def scheme_to_dp_result(setting: Sequence, scheme: Scheme, latency: float) -> dict:
    """One entry of ``dp_results.json`` (schema of latency_model.py:233-252)."""
    batch_slices = [b for b, _ in scheme]
    token_lists = {tuple(s) for _, s in scheme}
    if len(token_lists) != 1:
        raise AssertionError("every batch slice must use the same token slicing")
    return {"model_name": setting[0], "batch_size": setting[1], "model_parallel_size": setting[2],
            "pipeline_length": setting[3], "data_parallel_size": setting[4],
            "n_nodes": setting[5], "gpus_per_node": setting[6], "latency": latency,
            "batch_slices": batch_slices, "input_slices": list(next(iter(token_lists)))}


# model, batch, tp, pipeline length, dp, nodes, gpus per node: single 8xB200 box settings
B200_SETTINGS = [
    ("gpt3-1b", 8, 1, 8, 1, 1, 8),
    ("gpt3-1b", 8, 1, 4, 1, 1, 4),
    ("gpt3-1b", 8, 1, 2, 1, 1, 2),
    ("gpt3-13b", 8, 2, 4, 1, 1, 8),
    ("gpt3-44b", 4, 4, 2, 1, 1, 8),
]


def main(settings=None, data_dir="performance_model_data", out="dp_results.json", step_gap=None,
         kernel_model=False, fused_tp=True):
    """Schedules for ``settings`` written to ``out``.  With ``kernel_model`` the latency tables
    are not read from ``data_dir`` but synthesised from the analytic B200 kernel model
    (``kernel_model.py``) into a scratch directory; entries are tagged with their table's origin."""
    settings = settings or B200_SETTINGS
    results = []
    for s in settings:
        try:
            gap, table_dir = step_gap, data_dir
            if kernel_model:
                import tempfile
                from .kernel_model import write_tables
                table_dir = tempfile.mkdtemp(prefix="terapipe_tables_")
                gap = gap or 64
                write_tables(s[0], s[2], range(1, s[1] + 1), table_dir, step=gap,
                             fused_tp=fused_tp and s[2] > 1, total_batch=s[1])
            if gap is None:  # the granularity the table was measured with
                path = os.path.join(table_dir, f"latency_model.{s[0]}.mp_{s[2]}.json")
                lens = sorted({int(k.split("_")[1]) for k in json.load(open(path))})
                gap = min(b - a for a, b in zip(lens, lens[1:])) if len(lens) > 1 else STEP_GAP
            scheme, latency = analysis_model(*s[:4], data_dir=table_dir, step_gap=gap,
                                             verbose=not kernel_model)
        except FileNotFoundError as e:
            print(f"skip {s[0]}: {e}")
            continue
        if scheme is not None:
            entry = scheme_to_dp_result(s, scheme, latency)
            entry["table"] = "kernel-model" if kernel_model else "measured"
            results.append(entry)
    with open(out, "w") as f:
        json.dump(results, f, indent=4)
    return results


def auto_schedule(model_name, batch_size, tp, pp, fused_tp=True, step=64, n_layers=None):
    """(batch_slices, input_slices, predicted seconds) for one layout, planned on tables
    synthesised from the analytic B200 kernel model (no measurement files needed)."""
    import shutil
    import tempfile
    from .kernel_model import write_tables
    table_dir = tempfile.mkdtemp(prefix="terapipe_tables_")
    try:
        write_tables(model_name, tp, range(1, batch_size + 1), table_dir, step=step,
                     fused_tp=fused_tp and tp > 1, total_batch=batch_size)
        scheme, latency = analysis_model(model_name, batch_size, tp, pp, data_dir=table_dir,
                                         step_gap=step, n_layers=n_layers, verbose=False)
    finally:
        shutil.rmtree(table_dir, ignore_errors=True)
    if scheme is None:
        raise RuntimeError(f"no feasible schedule for {model_name} batch {batch_size} tp {tp} pp {pp}")
    return [b for b, _ in scheme], list(scheme[0][1]), latency


def cli(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="slice schedules from latency tables")
    ap.add_argument("--data-dir", default="performance_model_data")
    ap.add_argument("--out", default="dp_results.json")
    ap.add_argument("--step-gap", type=int, default=None)
    ap.add_argument("--kernel-model", action="store_true",
                    help="synthesise the tables from the analytic B200 kernel model")
    a = ap.parse_args(argv)
    return main(data_dir=a.data_dir, out=a.out, step_gap=a.step_gap, kernel_model=a.kernel_model)


if __name__ == "__main__":
    cli()
