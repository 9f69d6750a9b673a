#!/usr/bin/env python
"""Run one planned schedule from ``dp_results.json`` and record measured vs predicted latency
in ``dp_evaluation_results/dp_eval-<model>-<index>.json`` (skipped if the file exists).
Flags follow the reference tool (dp_slices_evaluation.py:13-22)."""
import argparse
import json
import os

import torch.distributed as dist

from terapipe_b200.models import TransformerConfig
from terapipe_b200.planner.memory_model import engine_memory_per_gpu
from terapipe_b200.runtime import cli
from terapipe_b200.runtime.runner import NCCLTransformerRunner


def main():
    parser = argparse.ArgumentParser(description="evaluate a planned slice schedule")
    cli.add_rank_arguments(parser)
    parser.add_argument("--model-name", type=str, default="gpt3-1b")
    parser.add_argument("--index", type=int, default=0)
    parser.add_argument("--n-steps", type=int, default=10)
    parser.add_argument("--mixed-precision", action="store_true", default=True)
    parser.add_argument("--verbose", action="store_true", default=False)
    parser.add_argument("--checkpoint-gradients", action="store_true", default=False)
    parser.add_argument("--dp-results", type=str, default="dp_results.json")
    parser.add_argument("--n-layers", type=int, default=None)
    parser.add_argument("--memory-limit", type=float, default=None)
    parser.add_argument("--tp-comm", default="fused", choices=["nccl", "fused", "sp"])
    args = parser.parse_args()
    cli.resolve_ranks(args)
    out_path = os.path.join("dp_evaluation_results", f"dp_eval-{args.model_name}-{args.index}.json")
    if os.path.exists(out_path):
        if args.rank == 0:
            print("already evaluated:", out_path)
        return
    with open(args.dp_results) as f:
        entries = [e for e in json.load(f) if e["model_name"] == args.model_name]
    e = entries[args.index]
    mp, pp, dp = e["model_parallel_size"], e["pipeline_length"], e["data_parallel_size"]
    assert dp * mp * pp == args.world_size, "world size does not match the planned layout"
    result = dict(e, n_gpus=args.world_size, n_steps=args.n_steps, rank=args.rank,
                  mixed_precision=args.mixed_precision, predicted_latency=e["latency"])
    limit = args.memory_limit if args.memory_limit is not None else cli.device_memory_gb()
    if engine_memory_per_gpu(args.model_name, e["batch_size"], tp=mp, pp=pp, n_layers=args.n_layers) > limit:
        result["mean_time"] = result["std_time"] = "OOM"
    else:
        config = TransformerConfig.from_predefined_model(args.model_name, n_devices=args.world_size,
                                                         batch_size=e["batch_size"],
                                                         n_layers=args.n_layers)
        runner = NCCLTransformerRunner(
            config, e["batch_slices"], e["input_slices"], f"tcp://{args.ip_address}:{args.port}",
            args.world_size, dp, mp, pp, args.rank, args.local_rank,
            mixed_precision=args.mixed_precision, init_process_group=args.world_size > 1,
            checkpoint_gradients=args.checkpoint_gradients, tp_comm=args.tp_comm)
        result["mean_time"], result["std_time"] = runner.run(args.n_steps, verbose=args.verbose)
    if args.rank == 0:
        os.makedirs("dp_evaluation_results", exist_ok=True)
        with open(out_path, "w") as f:
            json.dump(result, f, indent=2)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
