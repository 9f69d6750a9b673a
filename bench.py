#!/usr/bin/env python
"""Headline benchmark: training-iteration throughput of GPT-3-shaped decoder stacks.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...   (N > 1)

``value`` (every N): GPT3-1B shape (24 layers, hidden 2048, 16 heads, seq 2048), global batch 8,
fp16 mixed precision with fp32 master weights + Adam, 16 uniform token slices, pipeline = N
stages x tensor-parallel 1.  Synthetic N(0,1) inputs, random-init weights.  Total work is fixed
as N grows (strong scaling).

Further blocks ride in the same JSON line, each timed the same way with its own step count:

* N = 8: ``headline`` (GPT3-13B, pipeline 4 x tensor-parallel 2), ``headline_44b`` (GPT3-44B,
  pipeline 2 x tensor-parallel 4, batch 4) and ``headline_tp8`` (8 layers of GPT3-175B width,
  tensor-parallel 8, batch 2), with the fused GEMM + collective kernels;
* N = 2, 4: ``tp_block``: 4 layers of GPT3-13B width with tensor-parallel N, once per
  tensor-parallel communication mode (NCCL after the GEMM, fused all-reduce, sequence-parallel
  reduce-scatter / all-gather), with the relative error of the gradients against the NCCL mode.

Rank 0 prints ONE JSON line.  Times are CUDA events around exactly K steps after W >= 3 warm-up
steps, maximum over ranks; ``e2e`` repeats the measurement through ``Trainer.train_step`` with
the per-step host->device input copy (from pinned memory) and the device->host loss read inside
the timed region.

``--impl reference`` runs the unmodified reference (installed under ``baseline/_ref``) through
its own ``NCCLTransformerRunner.step`` on the same models, layouts and slices, block by block.

The further blocks run in child processes (one per rank, with a process group of their own) under
``--block-timeout`` seconds each: a block that fails or hangs is reported in its own entry
(``error`` / ``timed_out``) and cannot lose the numbers measured before it.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# No published single-box number exists for these configs: the reference's numbers are
# 192-384 V100 cluster latencies, so there is nothing to divide by.
BASELINE_TOKENS_PER_S = None

METRIC = "training throughput (tokens/s), GPT-3-shaped decoder, fwd+bwd+Adam per iteration"

# Extra blocks by GPU count.  `steps` caps the timed steps of the block (warm-up is always >= 3).
# In the order they run: the two named layouts first, so that a run that is cut short by its time
# budget loses the variations, not the named configurations.
HEADLINE_BLOCKS = {
    "headline": dict(model="gpt3-13b", batch=8, tp=2, pp=4, seq_slices=16, batch_slices=1, steps=5),
    "headline_44b": dict(model="gpt3-44b", batch=4, tp=4, pp=2, seq_slices=8, batch_slices=1,
                         steps=3, checkpoint_gradients=True),
    # the 13B layout with the batch / token slices chosen by the dynamic program over the B200
    # latency tables (both arms read the same committed schedule)
    "headline_planned": dict(model="gpt3-13b", batch=8, tp=2, pp=4, schedule="dp_results.json",
                             seq_slices=16, batch_slices=1, steps=5),
    "headline_tp8": dict(model="gpt3-175b", n_layers=8, batch=2, tp=8, pp=1, seq_slices=8,
                         batch_slices=1, steps=5),
}
TP_BLOCK = dict(model="gpt3-13b", n_layers=4, batch=8, pp=1, seq_slices=16, batch_slices=1, steps=5)


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
    ap.add_argument("--tp-comm", default="fused", choices=["nccl", "fused", "sp"])
    ap.add_argument("--dp-comm", default="nccl", choices=["nccl", "fused"])
    ap.add_argument("--no-graph", action="store_true", help="never capture the step in a CUDA graph")
    ap.add_argument("--graph", action="store_true", help="capture even when the stage communicates")
    ap.add_argument("--launch-plan", action="store_true",
                    help="stages that run eagerly replay recorded launch lists (see runtime/launch_plan.py)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--checkpoint-gradients", action="store_true",
                    help="reference arm: recompute the attention core in backward (this library always does)")
    ap.add_argument("--blocks", default="auto",
                    help="'auto' (the blocks of this GPU count), 'none', or a comma list of block names")
    ap.add_argument("--child-block", default=None, help=argparse.SUPPRESS)
    ap.add_argument("--total-budget", type=float, default=1500.0,
                    help="seconds after which no further block is started")
    ap.add_argument("--block-timeout", type=float, default=None,
                    help="seconds a single block may take (default 420 ours, 900 reference)")
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


class Deadline:
    """Host-side guard of one block: when the armed time runs out, rank 0 emits the JSON line
    with what exists and every rank ends its process with status 0."""

    def __init__(self, rank, emit):
        self.rank, self.emit = rank, emit
        self.until, self.label = None, None
        self.lock = threading.Lock()
        threading.Thread(target=self._watch, daemon=True).start()

    def arm(self, seconds, label):
        with self.lock:
            self.until, self.label = time.time() + seconds, label

    def disarm(self):
        with self.lock:
            self.until = None

    def _watch(self):
        while True:
            time.sleep(1.0)
            with self.lock:
                expired = self.until is not None and time.time() > self.until
                label = self.label
            if expired:
                if self.rank == 0:
                    self.emit(label)
                else:
                    time.sleep(3.0)
                sys.stdout.flush()
                os._exit(0)


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def config_dict(**kw):
    """The `config` object of a block; both arms fill the same keys."""
    keys = ("model", "n_layers", "hidden", "heads", "global_batch", "seq_len", "parallelism",
            "batch_slices", "seq_slices", "activation", "mixed_precision", "optimizer",
            "attention_recompute", "cuda_graph", "launch_plan", "tp_comm", "dp_comm", "l2")
    return {k: kw.get(k) for k in keys}


L2_NOTE = "per-step working set (weights + activations, several GB) far exceeds the 126 MB L2"


def slices_for(spec, seq_len, args=None):
    """(batch_slices, seq_slices) of a block: uniform, or from --schedule for the main block."""
    from terapipe_b200.utils import uniform_slice
    if args is not None and args.schedule == "auto":
        from terapipe_b200.planner.latency_model import auto_schedule
        bs, ss, _ = auto_schedule(spec["model"], spec["batch"], spec["tp"], spec["pp"],
                                  fused_tp=args.tp_comm != "nccl", n_layers=spec.get("n_layers"))
        return bs, ss
    if args is not None and args.schedule:
        with open(args.schedule) as f:
            sched = json.load(f)
        if isinstance(sched, list):
            match = [e for e in sched if e.get("model_name") == spec["model"] and
                     e.get("model_parallel_size") == spec["tp"] and
                     e.get("pipeline_length") == spec["pp"] and e.get("batch_size") == spec["batch"]]
            sched = match[0] if match else sched[args.schedule_index]
        return list(sched["batch_slices"]), list(sched["input_slices"])
    if spec.get("schedule"):
        # the entry the slice planner wrote for this model and layout (a committed dp_results file)
        with open(os.path.join(ROOT, spec["schedule"])) as f:
            for e in json.load(f):
                if (e.get("model_name") == spec["model"] and e.get("model_parallel_size") == spec["tp"]
                        and e.get("pipeline_length") == spec["pp"] and e.get("batch_size") == spec["batch"]):
                    return list(e["batch_slices"]), list(e["input_slices"])
        raise ValueError(f"no schedule for {spec['model']} in {spec['schedule']}")
    if "seq_slice_list" in spec:
        return list(spec["batch_slice_list"]), list(spec["seq_slice_list"])
    return (uniform_slice(spec["batch"], spec.get("batch_slices", 1)),
            uniform_slice(seq_len, spec["seq_slices"]))


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


# ---------------------------------------------------------------------------------------------
class OursArm:
    """This repository's engine through its public API (`Trainer`)."""
    name = "ours"

    def __init__(self, args):
        self.args = args

    def setup(self, rank, world, local):
        import torch
        import torch.distributed as dist
        self.rank, self.world, self.local = rank, world, local
        if not torch.cuda.is_available():
            return "no CUDA device (the engine is sm_100a only)"
        torch.cuda.set_device(local)
        self.device = torch.device("cuda", local)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.device)
        if self.args.launch_plan:
            os.environ["TERAPIPE_LAUNCH_PLAN"] = "1"
        return None

    def _trainer(self, spec, batch_slices, seq_slices, tp_comm):
        from terapipe_b200.runtime.trainer import Trainer
        a = self.args
        return Trainer(spec["model"], batch_size=spec["batch"], tp=spec["tp"], pp=spec["pp"],
                       batch_slices=batch_slices, seq_slices=seq_slices, dtype=a.dtype,
                       n_layers=spec.get("n_layers"), activation=a.activation or "gelu",
                       use_graph=(False if a.no_graph else (True if a.graph else None)),
                       tp_comm=tp_comm, dp_comm=a.dp_comm)

    def measure(self, spec, steps, warmup, main=False, tp_comm=None, keep_grads=False):
        import torch
        from terapipe_b200.models import MODEL_CONFIGS
        a = self.args
        seq_len = MODEL_CONFIGS[spec["model"]][2]
        batch_slices, seq_slices = slices_for(spec, seq_len, a if main else None)
        tp_comm = tp_comm or a.tp_comm
        torch.cuda.reset_peak_memory_stats()
        trainer = self._trainer(spec, batch_slices, seq_slices, tp_comm)
        eng = trainer.engine
        cfg = trainer.config
        tokens = cfg.batch_size * cfg.seq_len * trainer.topo.dp

        # ---- device-timed: inputs already resident, K steps
        trainer.load_input(trainer.synthetic_input(0))
        for _ in range(warmup):
            eng.step()
        launches0 = eng.launch_count
        sampler = ClockSampler(self.local)
        if self.rank == 0:
            sampler.start()
        ms = timed_steps(eng.step, steps, self.world, self.device)
        clocks = sampler.stop() if self.rank == 0 else None
        launches = eng.launch_count - launches0
        eng.check_status()
        ms_per_step = ms / steps

        # ---- end to end through the public API: pinned host input -> H2D, step, loss -> D2H
        e2e = None
        if not a.no_e2e:
            host_inputs = [trainer.synthetic_input(i, pinned=True) for i in range(2)]
            state = {"i": 0, "loss": None}

            def e2e_step():
                x = host_inputs[state["i"] % 2] if host_inputs[0] is not None else None
                state["loss"] = trainer.train_step(x)
                state["i"] += 1

            for _ in range(2):
                e2e_step()
            ms_e2e = timed_steps(e2e_step, steps, self.world, self.device)
            trainer.finish()
            h2d = cfg.seq_len * cfg.batch_size * cfg.embedding_dim * 2
            e2e = {"value": tokens / (ms_e2e / steps / 1e3), "unit": "tokens/s",
                   "ms_per_step": ms_e2e / steps, "h2d_bytes_per_step": h2d,
                   "d2h_bytes_per_step": 8, "last_loss": state["loss"]}
        grads = None
        if keep_grads:
            trainer.load_input(trainer.synthetic_input(0))
            eng.compute_grads()
            grads = eng.grad.clone()
        peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30
        value = tokens / (ms_per_step / 1e3)
        pp, tp, dp = trainer.topo.pp, trainer.topo.tp, trainer.topo.dp
        block = {
            "value": value, "unit": "tokens/s", "tokens_per_s": value, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "iteration_latency_s": ms_per_step / 1e3,
            "config": config_dict(
                model=spec["model"], n_layers=cfg.n_layers, hidden=cfg.embedding_dim,
                heads=cfg.num_attention_heads, global_batch=cfg.batch_size * dp, seq_len=cfg.seq_len,
                parallelism=f"pp{pp}xtp{tp}xdp{dp}", batch_slices=batch_slices, seq_slices=seq_slices,
                activation=cfg.activation, mixed_precision="fp32 master weights, loss scale 128",
                optimizer="fused mixed-precision Adam (this library)",
                attention_recompute=True, cuda_graph=("step" if eng.use_graph else
                                                      ("segments" if eng._seg_graphs is not None else False)),
                launch_plan=eng._plan is not None, tp_comm=eng.tp_comm, dp_comm=eng.dp_comm, l2=L2_NOTE),
            "gpu_launches": launches, "clocks": clocks, "e2e": e2e,
            "peak_memory_gb_torch_allocator": round(peak_gb, 2),
        }
        trainer.close()
        del trainer, eng
        gc.collect()
        torch.cuda.empty_cache()
        return (block, grads) if keep_grads else block

    def tp_block(self, spec, steps, warmup):
        """Tensor-parallel layer stack once per communication mode; gradients compared with the
        NCCL mode's."""
        import torch
        out = {"config": None, "modes": {}}
        ref_grads = None
        modes = ["nccl", "fused"]
        from terapipe_b200.runtime.engine import StageEngine
        if "sp" in getattr(StageEngine, "TP_COMM_MODES", ()):
            modes.append("sp")
        for mode in modes:
            print(f"[tp_block] rank {self.rank}: mode {mode}", file=sys.stderr, flush=True)
            block, grads = self.measure(spec, steps, warmup, tp_comm=mode, keep_grads=True)
            entry = {"ms_per_step": block["ms_per_step"], "tokens_per_s": block["value"],
                     "e2e_ms_per_step": block["e2e"]["ms_per_step"] if block["e2e"] else None,
                     "gpu_launches": block["gpu_launches"], "clocks": block["clocks"]}
            if ref_grads is None:
                ref_grads = grads
            else:
                num = (grads.double() - ref_grads.double()).norm() ** 2
                den = ref_grads.double().norm() ** 2
                t = torch.stack([num, den])
                if self.world > 1:
                    import torch.distributed as dist
                    dist.all_reduce(t)
                entry["grad_rel_err_vs_nccl"] = float((t[0] / t[1]).sqrt().item())
            out["modes"][mode] = entry
            if out["config"] is None or mode == self.args.tp_comm:
                out["config"] = block["config"]
            out["steps"], out["warmup"] = block["steps"], block["warmup"]
            del grads
        del ref_grads
        torch.cuda.empty_cache()
        return out

    def finish(self):
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
            dist.destroy_process_group()


def make_arm(args):
    if args.impl == "reference":
        from baseline.reference_arm import ReferenceArm
        return ReferenceArm(args, timed_steps, ClockSampler, slices_for, config_dict, L2_NOTE)
    return OursArm(args)


def main():
    args = parse_args()
    t_start = time.time()
    if args.child_block:
        return child_main(args)
    rank, world, local = dist_env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    warmup = max(args.warmup, 3)
    arm = make_arm(args)
    why = arm.setup(rank, world, local)
    if why is not None:
        if rank == 0:
            print(json.dumps({"impl": arm.name, "unavailable": why}), flush=True)
        # a reference arm that cannot be set up is a valid outcome; this repository's own arm is not
        sys.exit(0 if arm.name == "reference" else 1)

    out = {"metric": METRIC, "impl": arm.name, "n_gpus": world, "higher_is_better": True,
           "scaling": "strong", "dtype": args.dtype if arm.name == "ours" else "fp16"}
    printed = threading.Event()

    def emit(timed_out_label=None):
        if rank != 0 or printed.is_set():
            return
        printed.set()
        if timed_out_label is not None:
            out.setdefault(timed_out_label, {})
            if isinstance(out[timed_out_label], dict):
                out[timed_out_label]["timed_out"] = True
        print(json.dumps(out), flush=True)

    limit = args.block_timeout or (420.0 if arm.name == "ours" else 900.0)
    deadline = Deadline(rank, emit)

    main_spec = dict(model=args.model, n_layers=args.n_layers, batch=args.batch, tp=args.tp,
                     pp=args.pp if args.pp is not None else world // args.tp,
                     seq_slices=args.seq_slices, batch_slices=args.batch_slices,
                     checkpoint_gradients=args.checkpoint_gradients)
    deadline.arm(2 * limit, "main")
    blk = arm.measure(main_spec, args.steps, warmup, main=True)
    deadline.disarm()
    out.update({"value": blk["value"], "unit": "tokens/s", "steps": blk["steps"], "warmup": blk["warmup"],
                "ms_per_step": blk["ms_per_step"], "iteration_latency_s": blk["iteration_latency_s"],
                "vs_baseline": (blk["value"] / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
                "data": blk.get("data", "synthetic N(0,1) hidden states, random-init weights"),
                "config": blk["config"], "gpu_launches": blk["gpu_launches"], "clocks": blk["clocks"],
                "e2e": blk["e2e"]})
    if "peak_memory_gb_torch_allocator" in blk:
        out["peak_memory_gb_torch_allocator"] = blk["peak_memory_gb_torch_allocator"]

    # ---- further blocks
    default_main = (args.model == "gpt3-1b" and args.tp == 1 and args.pp is None and args.n_layers is None)
    if args.blocks == "auto":
        names = []
        if default_main and world == 8:
            names = list(HEADLINE_BLOCKS)
        elif default_main and world in (2, 4):
            names = ["tp_block"]
    elif args.blocks == "none":
        names = []
    else:
        names = [n for n in args.blocks.split(",") if n]
    # Every further block runs in child processes, one per rank, that form a process group of
    # their own: a block that faults, runs out of memory or hangs ends with its children and
    # costs only its own entry, never the numbers measured before it.
    arm.finish()                       # the parent's process group and device memory are released
    gc.collect()
    try:
        import torch
        torch.cuda.empty_cache()
    except Exception:  # noqa: BLE001
        pass
    base_port = int(os.environ.get("MASTER_PORT", "29500"))
    for i, name in enumerate(names):
        remaining = args.total_budget - (time.time() - t_start)
        if remaining < 60:
            out[name] = {"skipped": f"time budget of {args.total_budget:.0f} s for the whole run is used up"}
            continue
        if name != "tp_block" and HEADLINE_BLOCKS[name]["tp"] * HEADLINE_BLOCKS[name]["pp"] != world:
            out[name] = {"skipped": "needs %d GPUs" % (HEADLINE_BLOCKS[name]["tp"] * HEADLINE_BLOCKS[name]["pp"])}
            continue
        # torchrun's agent variables must not reach the children: with TORCHELASTIC_USE_AGENT_STORE
        # set, rank 0 would look for the agent's store on the new port instead of opening one
        env = {k: v for k, v in os.environ.items() if not k.startswith(("TORCHELASTIC_", "TORCH_NCCL_ASYNC"))}
        env.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(base_port + 101 + 7 * i),
                   RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(local))
        cmd = [sys.executable, os.path.abspath(__file__), "--child-block", name] + sys.argv[1:]
        entry = run_block_child(cmd, env, min(limit, remaining + 120), limit)
        if rank == 0:
            out[name] = entry
    emit()


def _last_json(text):
    """The last line of `text` that parses as a JSON object, or None."""
    if isinstance(text, bytes):
        text = text.decode(errors="replace")
    entry = None
    for line in (text or "").splitlines():
        if line.startswith("{"):
            try:
                entry = json.loads(line)
            except ValueError:
                pass
    return entry


def run_block_child(cmd, env, timeout, limit):
    """Run one further block as a child process and return its entry.  The child prints a JSON
    line whenever it has something complete (for a tensor-parallel block: after every
    communication mode), the last one counts; a child that is ended by the time limit or exits
    with an error after such a line keeps that result, with a note of what happened."""
    try:
        res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                             timeout=timeout)
        entry = _last_json(res.stdout)
        tail = (res.stderr or "").strip().splitlines()[-3:]
        if entry is None:
            entry = {"error": f"child exited with status {res.returncode}", "stderr_tail": tail}
        elif res.returncode != 0:
            entry["child_exit_status"] = res.returncode
            entry["stderr_tail"] = [ln[:200] for ln in tail]
    except subprocess.TimeoutExpired as e:
        err = e.stderr.decode(errors="replace") if isinstance(e.stderr, bytes) else (e.stderr or "")
        entry = _last_json(e.stdout) or {}
        entry.update({"timed_out": True, "limit_s": limit,
                      "stderr_tail": [ln[:200] for ln in err.strip().splitlines()[-12:]]})
    return entry


def child_main(args):
    """One further block in a process group of its own (see main); rank 0 prints the block."""
    import faulthandler
    limit = args.block_timeout or (420.0 if args.impl == "ours" else 900.0)
    # a block that hangs leaves the Python stack of every thread in its stderr before it is ended
    faulthandler.dump_traceback_later(max(30.0, 0.85 * limit), exit=False)
    rank, world, local = dist_env()
    warmup = max(args.warmup, 3)
    arm = make_arm(args)
    why = arm.setup(rank, world, local)
    if why is not None:
        if rank == 0:
            print(json.dumps({"unavailable": why}), flush=True)
        return
    name = args.child_block
    if name == "tp_block":
        spec = dict(TP_BLOCK, tp=world)
        entry = arm.tp_block(spec, min(args.steps, spec["steps"]), warmup)
    else:
        spec = dict(HEADLINE_BLOCKS[name])
        steps = min(args.steps, spec["steps"])
        if arm.name == "ours" and spec["tp"] > 1:
            # both fused tensor-parallel forms; the block reports the faster one and lists both
            modes = {}

            def summary():
                ok = {m: b for m, b in modes.items() if "ms_per_step" in b}
                best = min(ok, key=lambda m: ok[m]["ms_per_step"])
                e = dict(ok[best])
                e["tp_comm_modes"] = {m: ({"ms_per_step": b["ms_per_step"], "tokens_per_s": b["value"],
                                           "e2e_ms_per_step": (b["e2e"] or {}).get("ms_per_step")}
                                          if "ms_per_step" in b else b) for m, b in modes.items()}
                return e

            failed = None
            for mode in ("fused", "sp"):
                try:
                    modes[mode] = arm.measure(spec, steps, warmup, tp_comm=mode)
                except ValueError as e:      # raised identically on every rank before any kernel runs
                    modes[mode] = {"skipped": str(e)[:200]}
                except Exception as e:       # noqa: BLE001 - the ranks may be out of step now: stop here
                    modes[mode] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
                    failed = e
                if rank == 0 and any("ms_per_step" in b for b in modes.values()):
                    print(json.dumps(summary()), flush=True)     # the parent keeps the last line
                if failed is not None:
                    break
            if failed is not None:
                if not any("ms_per_step" in b for b in modes.values()):
                    raise failed
                sys.stdout.flush()
                os._exit(3)                  # no collective teardown with ranks that may be elsewhere
            entry = summary()
        else:
            entry = arm.measure(spec, steps, warmup)
    if rank == 0:
        print(json.dumps(entry), flush=True)
    arm.finish()


if __name__ == "__main__":
    main()
