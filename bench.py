#!/usr/bin/env python
"""Headline benchmark: training-iteration throughput of a GPT-3-shaped decoder stack.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...   (N > 1)

Default workload (every N): GPT3-1B shape (24 layers, hidden 2048, 16 heads, seq 2048),
global batch 8, fp16 mixed precision with fp32 master weights + Adam, 16 uniform token
slices, pipeline = N stages x tensor-parallel 1.  Synthetic N(0,1) inputs, random-init
weights.  Total work is fixed as N grows (strong scaling).  ``--model gpt3-13b --tp 2 --pp 4``
etc. select the larger layouts on 8 GPUs.

Rank 0 prints ONE JSON line.  ``value`` is tokens/s of the whole job, timed on the device
(CUDA events, max over ranks) over exactly K steps after W warm-up steps; ``e2e`` repeats
the measurement through ``Trainer.train_step`` with the per-step host->device input copy
(from pinned memory) and device->host loss read inside the timed region.

``--impl reference`` runs the unmodified reference (installed under ``baseline/_ref``)
through its own ``NCCLTransformerRunner.step`` on the same model/config/slices.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# No published single-box number exists for these configs: the reference's numbers are
# 192-384 V100 cluster latencies, so there is nothing to divide by.
BASELINE_TOKENS_PER_S = None


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt3-1b")
    ap.add_argument("--n-layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=None)
    ap.add_argument("--seq-slices", type=int, default=16)
    ap.add_argument("--batch-slices", type=int, default=1)
    ap.add_argument("--schedule", default=None,
                    help="JSON file with batch_slices / input_slices lists, a dp_results.json list, "
                         "or 'auto' (dynamic program over the B200 kernel model)")
    ap.add_argument("--schedule-index", type=int, default=0, help="entry of a dp_results.json list")
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--activation", default=None, choices=[None, "gelu", "relu"])
    ap.add_argument("--tp-comm", default="nccl", choices=["nccl", "fused"])
    ap.add_argument("--dp-comm", default="nccl", choices=["nccl", "fused"])
    ap.add_argument("--no-graph", action="store_true", help="never capture the step in a CUDA graph")
    ap.add_argument("--graph", action="store_true", help="capture even when the stage communicates")
    ap.add_argument("--launch-plan", action="store_true",
                    help="stages that run eagerly replay recorded launch lists (see runtime/launch_plan.py)")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def slices_from_args(args, seq_len):
    from terapipe_b200.utils import uniform_slice
    if args.schedule == "auto":
        # planned for this model and layout on kernel-model tables (every rank computes the same)
        from terapipe_b200.planner.latency_model import auto_schedule
        world = int(os.environ.get("WORLD_SIZE", "1"))
        pp = args.pp if args.pp is not None else world // args.tp
        bs, ss, _ = auto_schedule(args.model, args.batch, args.tp, pp, fused_tp=args.tp_comm == "fused",
                                  n_layers=args.n_layers)
        return bs, ss
    if args.schedule:
        with open(args.schedule) as f:
            sched = json.load(f)
        if isinstance(sched, list):
            # a dp_results list: the entry planned for this model and layout if there is one,
            # otherwise the entry at --schedule-index
            world = int(os.environ.get("WORLD_SIZE", "1"))
            pp = args.pp if args.pp is not None else world // args.tp
            match = [e for e in sched if e.get("model_name") == args.model and
                     e.get("model_parallel_size") == args.tp and e.get("pipeline_length") == pp and
                     e.get("batch_size") == args.batch]
            sched = match[0] if match else sched[args.schedule_index]
        return list(sched["batch_slices"]), list(sched["input_slices"])
    return uniform_slice(args.batch, args.batch_slices), uniform_slice(seq_len, args.seq_slices)


def max_over_ranks(value, world, device):
    import torch
    import torch.distributed as dist
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(world):
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def timed_steps(step_fn, steps, world, device):
    """K calls of step_fn between two CUDA events, barrier + synchronize on both sides."""
    import torch
    barrier_sync(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    e1.record()
    barrier_sync(world)
    return max_over_ranks(e0.elapsed_time(e1), world, device)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from terapipe_b200.models import MODEL_CONFIGS
    from terapipe_b200.runtime.trainer import Trainer

    rank, world, local = dist_env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    pp = args.pp if args.pp is not None else world // args.tp
    if args.launch_plan:
        os.environ["TERAPIPE_LAUNCH_PLAN"] = "1"
    seq_len = MODEL_CONFIGS[args.model][2]
    batch_slices, seq_slices = slices_from_args(args, seq_len)
    trainer = Trainer(args.model, batch_size=args.batch, tp=args.tp, pp=pp,
                      batch_slices=batch_slices, seq_slices=seq_slices,
                      dtype=args.dtype, n_layers=args.n_layers, activation=args.activation or "gelu",
                      use_graph=(False if args.no_graph else (True if args.graph else None)),
                      tp_comm=args.tp_comm, dp_comm=args.dp_comm)
    cfg = trainer.config
    tokens = cfg.batch_size * cfg.seq_len * trainer.topo.dp

    # ---- device-timed: inputs already resident, K steps
    trainer.load_input(trainer.synthetic_input(0))
    for _ in range(max(args.warmup, 3)):
        trainer.engine.step()
    launches0 = trainer.engine.launch_count
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed_steps(trainer.engine.step, args.steps, world, device)
    clocks = sampler.stop() if rank == 0 else None
    launches = trainer.engine.launch_count - launches0
    trainer.engine.check_status()
    ms_per_step = ms / args.steps

    # ---- end to end through the public API: pinned host input -> H2D, step, loss -> D2H
    e2e = None
    if not args.no_e2e:
        host_inputs = [trainer.synthetic_input(i, pinned=True) for i in range(2)]
        state = {"i": 0, "loss": None}

        def e2e_step():
            x = host_inputs[state["i"] % 2] if host_inputs[0] is not None else None
            state["loss"] = trainer.train_step(x)
            state["i"] += 1

        for _ in range(2):
            e2e_step()
        ms_e2e = timed_steps(e2e_step, args.steps, world, device)
        h2d = cfg.seq_len * cfg.batch_size * cfg.embedding_dim * 2
        e2e = {"value": tokens / (ms_e2e / args.steps / 1e3), "unit": "tokens/s",
               "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 4, "last_loss": state["loss"]}

    if rank == 0:
        value = tokens / (ms_per_step / 1e3)
        out = {
            "metric": "training throughput (tokens/s), GPT-3-shaped decoder, fwd+bwd+Adam per iteration",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "iteration_latency_s": ms_per_step / 1e3,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
            "dtype": args.dtype, "data": "synthetic N(0,1) hidden states, random-init weights",
            "impl": "ours",
            "config": {"model": args.model, "n_layers": cfg.n_layers, "hidden": cfg.embedding_dim,
                       "heads": cfg.num_attention_heads, "global_batch": cfg.batch_size * trainer.topo.dp,
                       "seq_len": cfg.seq_len, "parallelism": f"pp{pp}xtp{args.tp}xdp{trainer.topo.dp}",
                       "batch_slices": batch_slices, "seq_slices": seq_slices,
                       "activation": cfg.activation, "mixed_precision": "fp32 master + Adam, loss scale 128",
                       "cuda_graph": bool(trainer.engine.use_graph),
                       "launch_plan": trainer.engine._plan is not None, "tp_comm": trainer.engine.tp_comm, "dp_comm": trainer.engine.dp_comm,
                       "l2": "per-step working set (weights + activations, several GB) far exceeds the 126 MB L2"},
            "gpu_launches": launches, "clocks": clocks, "e2e": e2e,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    from baseline.reference_arm import run as run_ref
    run_ref(args, dist_env, timed_steps, ClockSampler, slices_from_args)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
