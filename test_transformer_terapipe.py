#!/usr/bin/env python
"""Production driver: sweeps (tensor parallel, pipeline parallel, batch, batch slices, token
slices) given as comma lists, times training iterations, writes ``results.json`` on rank 0.
Same flags as the reference driver (test_transformer_terapipe.py:359-377) plus ``--n-layers``,
``--memory-limit`` (GB, default: the device's capacity) and ``--tp-comm``.
"""
import argparse
import gc
import json
import time
from itertools import product

import torch

from terapipe_b200.models import MODEL_CONFIGS, TransformerConfig
from terapipe_b200.planner.memory_model import engine_memory_per_gpu
from terapipe_b200.runtime import cli
from terapipe_b200.runtime.cli import parse_comma_delimited_arg  # noqa: F401
from terapipe_b200.runtime.runner import (LOSS_SCALE_FACTOR, NCCLTransformer,  # noqa: F401
                                          NCCLTransformerRunner)
from terapipe_b200.utils import TimeoutError, uniform_slice


def main():
    parser = argparse.ArgumentParser(description="token-level pipeline + tensor parallel sweep")
    cli.add_rank_arguments(parser)
    for flag in ("--model-parallel-size", "--pipeline-parallel-size", "--batch-size",
                 "--n-batch-slices", "--n-input-slices"):
        parser.add_argument(flag, metavar="N", type=str, default="1")
    parser.add_argument("--model", metavar="NAME", type=str, default="test", choices=cli.model_choices())
    parser.add_argument("--n-layers", type=int, default=None)
    parser.add_argument("--n-steps", metavar="N", type=int, default=10)
    parser.add_argument("--mixed-precision", action="store_true", default=False)
    parser.add_argument("--verify", action="store_true", default=False)
    parser.add_argument("--verbose", action="store_true", default=False)
    parser.add_argument("--checkpoint-gradients", action="store_true", default=False)
    parser.add_argument("--memory-limit", type=float, default=None)
    parser.add_argument("--tp-comm", default="fused", choices=["nccl", "fused", "sp"])
    args = parser.parse_args()
    cli.resolve_ranks(args)
    as_ints = lambda s: cli.parse_comma_delimited_arg(s, int)  # noqa: E731
    limit = args.memory_limit if args.memory_limit is not None else cli.device_memory_gb()
    results, init_group = [], True
    for mp, pp, batch, nbs, nis in product(as_ints(args.model_parallel_size),
                                           as_ints(args.pipeline_parallel_size),
                                           as_ints(args.batch_size), as_ints(args.n_batch_slices),
                                           as_ints(args.n_input_slices)):
        t_setup = time.time()
        if batch % nbs != 0 or args.world_size % (mp * pp) != 0:
            continue
        dp = args.world_size // (mp * pp)
        result = {"model": args.model, "n_gpus": args.world_size, "batch_size": batch,
                  "n_batch_slices": nbs, "n_input_slices": nis, "n_steps": args.n_steps,
                  "mixed_precision": args.mixed_precision, "model_parallel_size": mp,
                  "pipeline_parallel_size": pp, "rank": args.rank, "data_parallel_size": dp}
        need = engine_memory_per_gpu(args.model, batch, tp=mp, pp=pp, n_layers=args.n_layers)
        if need > limit:
            result["mean_time"] = result["std_time"] = "OOM"
            results.append(result)
            continue
        config = TransformerConfig.from_predefined_model(args.model, n_devices=args.world_size,
                                                         batch_size=batch, n_layers=args.n_layers)
        runner = NCCLTransformerRunner(
            config, uniform_slice(batch, nbs), uniform_slice(config.seq_len, nis),
            f"tcp://{args.ip_address}:{args.port}", args.world_size, dp, mp, pp, args.rank,
            args.local_rank, mixed_precision=args.mixed_precision, use_mpi=args.use_mpi,
            init_process_group=init_group and args.world_size > 1,
            checkpoint_gradients=args.checkpoint_gradients, tp_comm=args.tp_comm)
        init_group = False
        gc.collect()
        if args.rank == 0:
            print(f"-------- Beginning run for model {args.model}; using {args.world_size} GPUs; "
                  f"batch size {batch}; batch slices {nbs}; input slices {nis}; steps {args.n_steps}; "
                  f"mixed precision {args.mixed_precision}; model parallel size {mp}; "
                  f"pipeline parallel size {pp} --------", flush=True)
            print(f"-------- Experiment setup took {int((time.time() - t_setup) * 1000)} ms --------",
                  flush=True)
        try:
            if args.verify:
                runner.verify()
            else:
                mean_time, std_time = runner.run(args.n_steps, verbose=args.verbose)
                result["mean_time"], result["std_time"] = mean_time, std_time
                # beyond the reference's schema: job throughput, device-timed step of the slowest
                # rank, this rank's peak memory
                result["tokens_per_s"] = batch * dp * config.seq_len / mean_time
                result["max_over_ranks_device_ms"] = runner.max_over_ranks_device_ms()
                result["peak_memory_gb"] = runner.last_peak_memory_gb
        except (torch.cuda.OutOfMemoryError, TimeoutError) as e:
            print(e, flush=True)
            result["mean_time"] = result["std_time"] = "OOM"
        results.append(result)
        with open(f"results.rank{args.rank}.jsonl", "a") as f:  # one line per run and rank
            f.write(json.dumps(result) + "\n")
        del runner
        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    if args.rank == 0:
        with open("results.json", "w") as f:
            json.dump(results, f)
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
