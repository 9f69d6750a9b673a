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


def p2p_communication_latency(payload_size, group=None):
    """(mean, std) one-way latency in seconds of a ``payload_size``-element fp16 message between
    ranks 0 and 1 (name of the reference tool's measurement, p2p_comm_latency.py:14-32)."""
    return measure(payload_size, dist.get_rank(group) if group is not None else dist.get_rank())


def benchmark_p2p_communication(mpi_comm, rank, model_name, size_gap=32, batch_size=None,
                                out_dir="performance_model_data"):
    """Measure the stage-to-stage link for every message size of ``model_name`` and write
    ``<model>.communication_latency.json`` (sizes in tokens).  ``mpi_comm`` and ``size_gap`` are
    accepted for compatibility with the reference signature and not used: ranks come from
    ``torch.distributed`` and the sizes from :func:`token_sizes`."""
    _, hidden, seq_len, _ = MODEL_CONFIGS[model_name]
    batch = batch_size or BATCH_CONFIGS.get(model_name, 8)
    sizes = token_sizes(seq_len * batch)
    means, stds = [], []
    for tokens in sizes:
        if rank < 2:
            m, s = measure(tokens * hidden, rank)
            means.append(m)
            stds.append(s)
        dist.barrier()
    result = {"tensor_sizes": sizes, "mean": means, "std": stds}
    if rank == 0:
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, f"{model_name}.communication_latency.json"), "w") as f:
            json.dump(result, f)
    return result


def get_local_ip_address():
    """Single-machine launches rendezvous on the loopback address."""
    return "127.0.0.1"


def main():
    parser = argparse.ArgumentParser(description="stage-to-stage link latency")
    cli.add_rank_arguments(parser)
    parser.add_argument("--model", type=str, default="gpt3-1b", choices=cli.model_choices())
    parser.add_argument("--batch-size", type=int, default=None)
    parser.add_argument("--out-dir", type=str, default="performance_model_data")
    args = parser.parse_args()
    cli.resolve_ranks(args)
    init_distributed(f"tcp://{args.ip_address}:{args.port}", args.world_size, args.rank, args.local_rank)
    res = benchmark_p2p_communication(None, args.rank, args.model, batch_size=args.batch_size,
                                      out_dir=args.out_dir)
    if args.rank == 0:
        print("tokens, latency_us:",
              [(t, round(m * 1e6, 1)) for t, m in zip(res["tensor_sizes"], res["mean"])][-4:], flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
