#!/usr/bin/env python
"""Measure the single-layer latency table used by the slice planner.

For one layer (tensor parallel over ``--model-parallel-size`` ranks, no pipeline) and one token
slice, times forward, backward and optimizer update on the device for a grid of
``(batch, slice_len, context_len)`` and writes
``performance_model_data/latency_model.<model>.mp_<mp>.json`` (keys ``"b_s_c"``; fields
``{py_forward,forward,py_backward,backward,update}_{mean,std}`` plus ``wgrad_per_token_*``:
the engine computes weight gradients once per iteration over all rows, so their cost is
reported per token instead of inside ``backward``).  Existing keys are skipped,
so an interrupted run resumes; the file is flushed every ``--flush-every`` points.  Flags follow
the reference tool (terapipe_latency_model.py:120-141); ``--step-gap`` / ``--scan-grid`` choose
a coarser grid than its (8, (16,16,4)).
"""
import argparse
import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from terapipe_b200.models import BATCH_CONFIGS, MODEL_CONFIGS, TransformerConfig
from terapipe_b200.runtime import cli
from terapipe_b200.runtime.runner import init_distributed
from terapipe_b200 import parallel as mpu


def parse_json(r):
    """Table keys ``"b_s_c"`` -> ``(b, s, c)`` (terapipe_latency_model.py:103-108)."""
    return {tuple(int(v) for v in k.split("_")): val for k, val in r.items()}


def format_json(r):
    """Inverse of :func:`parse_json` (terapipe_latency_model.py:111-116)."""
    return {"_".join(str(v) for v in k): val for k, val in r.items()}


class TerapipeLatencyModel:
    """One layer, one slice: the slice of ``seqlen`` tokens attends to ``ctx`` cached rows."""

    def __init__(self, model_name, batch_size, seqlen, ctx, mixed_precision=True, tp_comm="fused", reps=4):
        self.reps = reps
        from terapipe_b200.runtime.engine import StageEngine
        cfg = TransformerConfig.from_predefined_model(model_name, batch_size=batch_size, n_layers=1)
        cfg.seq_len = ctx + seqlen
        slices = ([ctx] if ctx else []) + [seqlen]
        self.engine = StageEngine(cfg, [batch_size], slices, init="device", use_graph=False,
                                  tp_comm=tp_comm, segment_graphs=False)
        self.engine.set_input(torch.randn(cfg.seq_len, batch_size, cfg.embedding_dim))
        self.target = self.engine.slices[0][-1]

    def step(self):
        e = self.engine
        e._refresh_handles()
        if e.ar is not None:
            e.lib.tp_advance_counter(e.ar_epoch_base.data_ptr(), e._ar_calls_per_step, e._stream)
            e._ar_calls = 0
        if getattr(e, "sp", False):
            raise ValueError("the latency table is measured with tp_comm 'fused' or 'nccl'")
        # Steady state, not launch-bound: inside a training step the launches of a slice are
        # replayed from a CUDA graph, so the device never waits for the host.  Here every timed
        # phase is repeated `reps` times behind a short device-side sleep that lets the host
        # queue all launches first; the events then measure back-to-back kernel time.
        reps = self.reps
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        t0 = time.time()
        torch.cuda._sleep(400_000 * reps)
        ev[0].record()
        for _ in range(reps):
            e._forward_slice(self.target)
        ev[1].record()
        py_fwd = (time.time() - t0) / reps
        t0 = time.time()
        torch.cuda._sleep(600_000 * reps)
        ev[2].record()
        for _ in range(reps):
            e._backward_slice(self.target)
        ev[3].record()
        py_bwd = (time.time() - t0) / reps
        # weight gradients run once per iteration over all rows, not per slice: they are timed
        # apart and reported per token so the planner can add them as a per-layer constant
        e._weight_grads()
        ev[4].record()
        e._reduce_and_update()
        ev[5].record()
        torch.cuda.synchronize()
        return (py_fwd, ev[0].elapsed_time(ev[1]) / 1e3 / reps, py_bwd,
                ev[2].elapsed_time(ev[3]) / 1e3 / reps, ev[4].elapsed_time(ev[5]) / 1e3,
                ev[3].elapsed_time(ev[4]) / 1e3 / e.rows)

    def run(self, n_steps=10, warmup_steps=5):
        # the prefix rows must hold valid keys/values: run the context slice once
        e = self.engine
        e._refresh_handles()
        for sl in e.slices[0][:-1]:
            e._forward_slice(sl)
        rows = [self.step() for _ in range(n_steps + warmup_steps)][warmup_steps:]
        arr = np.array(rows)
        names = ("py_forward", "forward", "py_backward", "backward", "update", "wgrad_per_token")
        out = {}
        for i, n in enumerate(names):
            out[n + "_mean"] = float(arr[:, i].mean())
            out[n + "_std"] = float(arr[:, i].std())
        return out


def scan_points(model, batch_size, step_gap, scan_grid, batches=None):
    _, _, L, _ = MODEL_CONFIGS[model]
    nb, ns, nc = scan_grid
    if batches is None:
        batches = sorted({max(1, round(batch_size * (i + 1) / nb)) for i in range(nb)}) \
            if batch_size > 8 else list(range(1, batch_size + 1))
    seqs = sorted({max(step_gap, (L * (i + 1) // ns) // step_gap * step_gap) for i in range(ns)})
    ctxs = sorted({(L * (i + 1) // nc) // step_gap * step_gap for i in range(nc)})
    pts = {(b, s, c) for b in batches for s in seqs for c in ctxs if s + c <= L}
    pts |= {(b, s, 0) for b in batches for s in range(step_gap, L + 1, step_gap)}
    return pts


def main():
    parser = argparse.ArgumentParser(description="single-layer latency table")
    cli.add_rank_arguments(parser)
    parser.add_argument("--model", type=str, default="gpt3-1b", choices=cli.model_choices())
    parser.add_argument("--model-parallel-size", type=int, default=1)
    parser.add_argument("--pipeline-parallel-size", type=int, default=1)
    parser.add_argument("--batch-size", type=int, default=None)
    parser.add_argument("--n-batch-slices", type=int, default=1)
    parser.add_argument("--n-input-slices", type=int, default=1)
    parser.add_argument("--n-steps", type=int, default=10)
    parser.add_argument("--warmup-steps", type=int, default=5)
    parser.add_argument("--mixed-precision", action="store_true", default=True)
    parser.add_argument("--sort-function", type=int, default=0, choices=[0, 1, 2])
    parser.add_argument("--step-gap", type=int, default=64)
    parser.add_argument("--scan-grid", type=str, default="4,8,4")
    parser.add_argument("--flush-every", type=int, default=100)
    parser.add_argument("--max-points", type=int, default=None)
    parser.add_argument("--batches", type=str, default=None,
                        help="comma list of batch sizes to scan instead of the default set")
    parser.add_argument("--out-dir", type=str, default="performance_model_data")
    parser.add_argument("--tp-comm", default="fused", choices=["nccl", "fused", "sp"])
    args = parser.parse_args()
    cli.resolve_ranks(args)
    if args.world_size > 1:
        init_distributed(f"tcp://{args.ip_address}:{args.port}", args.world_size, args.rank, args.local_rank)
        mpu.initialize_model_parallel(args.model_parallel_size, 1, verbose=False)
    elif torch.cuda.is_available():
        torch.cuda.set_device(args.local_rank)
    batch = args.batch_size or BATCH_CONFIGS.get(args.model, 8)
    os.makedirs(args.out_dir, exist_ok=True)
    path = os.path.join(args.out_dir, f"latency_model.{args.model}.mp_{args.model_parallel_size}.json")
    table = json.load(open(path)) if os.path.exists(path) else {}
    grid = tuple(int(v) for v in args.scan_grid.split(","))
    only = [int(v) for v in args.batches.split(",")] if args.batches else None
    todo = [p for p in scan_points(args.model, batch, args.step_gap, grid, only)
            if "_".join(map(str, p)) not in table]
    # cheapest first, so that an out-of-memory point comes last (three alternative cost orders)
    keyfn = [lambda p: p[0] * p[1] * (p[1] + p[2]), lambda p: p[0] * (p[1] + p[2]),
             lambda p: p[0] * p[1]][args.sort_function]
    todo.sort(key=keyfn)
    if args.max_points:
        stride = max(1, len(todo) // args.max_points)
        todo = todo[::stride]

    def flush():
        if args.rank == 0:
            tmp = path + ".tmp"
            with open(tmp, "w") as f:
                json.dump(table, f)
            os.replace(tmp, path)

    for i, (b, s, c) in enumerate(todo):
        try:
            m = TerapipeLatencyModel(args.model, b, s, c, tp_comm=args.tp_comm)
            table[f"{b}_{s}_{c}"] = m.run(args.n_steps, args.warmup_steps)
            m.engine.close()      # unmaps the peer buffers of this point (collective)
            del m
        except torch.cuda.OutOfMemoryError:
            flush()
            raise
        if (i + 1) % args.flush_every == 0:
            flush()
    flush()
    if args.rank == 0:
        print(f"{len(table)} points in {path}", flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
