#!/usr/bin/env python
"""Grid runner: launches ``mpirun_terapipe.sh`` once per setting, each with a time limit, and
keeps the to-do list in ``experiments_remaining.json`` so that an interrupted sweep resumes.
Flags follow the reference tool (batch_test.py:50-61).  A run that exceeds the limit is ended
by the launcher, which stops only the processes it started."""
import argparse
import json
import os
import subprocess
from itertools import product

from terapipe_b200.planner.memory_model import engine_memory_per_gpu
from terapipe_b200.runtime import cli
from terapipe_b200.runtime.cli import parse_comma_delimited_arg  # noqa: F401

TODO_FILE = "experiments_remaining.json"


def run_experiment(exp, n_nodes, n_gpus, n_steps, extra, time_limit=500):
    model, mp, pp, batch, nbs, nis = exp
    cmd = ["bash", os.path.join(os.path.dirname(os.path.abspath(__file__)), "mpirun_terapipe.sh"),
           str(n_nodes), str(n_gpus), str(mp), str(pp), model, str(batch), str(nbs), str(nis),
           str(n_steps), *extra]
    env = dict(os.environ, MKL_THREADING_LAYER="GNU", TERAPIPE_TIME_LIMIT=str(time_limit))
    try:
        return subprocess.run(cmd, env=env, timeout=time_limit + 60).returncode
    except subprocess.TimeoutExpired:
        return 124


def main():
    parser = argparse.ArgumentParser(description="sweep over models and parallel layouts")
    parser.add_argument("--n-nodes", type=int, default=1)
    parser.add_argument("--n-gpus-per-node", type=int, default=8)
    for flag in ("--model-parallel-size", "--pipeline-parallel-size", "--batch-size",
                 "--n-batch-slices", "--n-input-slices"):
        parser.add_argument(flag, type=str, default="1")
    parser.add_argument("--model", type=str, default="gpt3-1b")
    parser.add_argument("--n-steps", type=int, default=10)
    parser.add_argument("--mixed-precision", action="store_true", default=False)
    parser.add_argument("--checkpoint-gradients", action="store_true", default=False)
    parser.add_argument("--memory-limit", type=float, default=None)
    parser.add_argument("--dry-run", action="store_true", default=False)
    args = parser.parse_args()
    ints = lambda s: cli.parse_comma_delimited_arg(s, int)  # noqa: E731
    limit = args.memory_limit if args.memory_limit is not None else cli.device_memory_gb()
    world = args.n_nodes * args.n_gpus_per_node
    if os.path.exists(TODO_FILE):
        todo = [tuple(e) for e in json.load(open(TODO_FILE))]
    else:
        todo = []
        for exp in product(args.model.split(","), ints(args.model_parallel_size),
                           ints(args.pipeline_parallel_size), ints(args.batch_size),
                           ints(args.n_batch_slices), ints(args.n_input_slices)):
            model, mp, pp, batch, nbs, _ = exp
            if world % (mp * pp) or batch % nbs:
                continue
            if engine_memory_per_gpu(model, batch, tp=mp, pp=pp) > limit:
                continue
            todo.append(exp)
    extra = (["--mixed-precision"] if args.mixed_precision else []) + \
            (["--checkpoint-gradients"] if args.checkpoint_gradients else [])
    while todo:
        with open(TODO_FILE, "w") as f:
            json.dump(todo, f)
        exp = todo[0]
        print("running", exp, flush=True)
        if not args.dry_run:
            run_experiment(exp, args.n_nodes, args.n_gpus_per_node, args.n_steps, extra)
        todo = todo[1:]
    if os.path.exists(TODO_FILE):
        os.remove(TODO_FILE)


if __name__ == "__main__":
    main()
