#!/usr/bin/env python
"""Point-to-point latency between two GPUs of this box (the inter-stage link of the pipeline).

Ranks 0 and 1 ping-pong a 16-bit buffer of ``tokens x hidden`` elements with NCCL send/recv;
the one-way latency is half the round trip, timed with CUDA events.  Writes
``performance_model_data/<model>.communication_latency.json`` with ``tensor_sizes`` (tokens),
``mean`` and ``std`` (seconds), the format the planner reads.  On NVSwitch every GPU pair is
equivalent, so one pair is measured (the reference measured the cross-node pair of a 2-node
cluster, p2p_comm_latency.py:14-52).
"""
import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from terapipe_b200.models import BATCH_CONFIGS, MODEL_CONFIGS
from terapipe_b200.runtime import cli
from terapipe_b200.runtime.runner import init_distributed


def token_sizes(max_tokens):
    sizes, t = [], 1
    while t < max_tokens:
        sizes.append(t)
        t = t * 2 if t < 1024 else int(t * 1.5)
    sizes.append(max_tokens)
    return sorted(set(sizes))


def measure(n_elems, rank, dtype=torch.float16):
    buf = torch.zeros(n_elems, dtype=dtype, device="cuda")
    steps = int(np.clip(30 - np.log2(max(n_elems, 1)), 3, 30))
    times = []
    for i in range(2 * steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if rank == 0:
            dist.send(buf, 1)
            dist.recv(buf, 1)
        else:
            dist.recv(buf, 0)
            dist.send(buf, 0)
        e1.record()
        torch.cuda.synchronize()
        if i >= steps:
            times.append(e0.elapsed_time(e1) / 2e3)
    return float(np.mean(times)), float(np.std(times))


def main():
    parser = argparse.ArgumentParser(description="stage-to-stage link latency")
    cli.add_rank_arguments(parser)
    parser.add_argument("--model", type=str, default="gpt3-1b", choices=cli.model_choices())
    parser.add_argument("--batch-size", type=int, default=None)
    parser.add_argument("--out-dir", type=str, default="performance_model_data")
    args = parser.parse_args()
    cli.resolve_ranks(args)
    init_distributed(f"tcp://{args.ip_address}:{args.port}", args.world_size, args.rank, args.local_rank)
    _, hidden, seq_len, _ = MODEL_CONFIGS[args.model]
    batch = args.batch_size or BATCH_CONFIGS.get(args.model, 8)
    sizes = token_sizes(seq_len * batch)
    means, stds = [], []
    for tokens in sizes:
        if args.rank < 2:
            m, s = measure(tokens * hidden, args.rank)
            means.append(m)
            stds.append(s)
        dist.barrier()
    if args.rank == 0:
        os.makedirs(args.out_dir, exist_ok=True)
        with open(os.path.join(args.out_dir, f"{args.model}.communication_latency.json"), "w") as f:
            json.dump({"tensor_sizes": sizes, "mean": means, "std": stds}, f)
        print("tokens, latency_us:", [(t, round(m * 1e6, 1)) for t, m in zip(sizes, means)][-4:], flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
