"""Shared command-line plumbing of the experiment drivers."""
from __future__ import annotations

import argparse
import os
from typing import Callable, List

from ..models import MODEL_CONFIGS


def add_rank_arguments(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("ip_address", type=str, help="the IP address of the head node")
    parser.add_argument("-p", "--port", type=int, default=7777, help="the port of the head node")
    parser.add_argument("--rank", metavar="I", type=int, default=None)
    parser.add_argument("--local-rank", metavar="I", type=int, default=None)
    parser.add_argument("--world-size", metavar="N", type=int, default=None)
    parser.add_argument("--use-mpi", action="store_true", default=False)


def resolve_ranks(args) -> None:
    """Ranks from ``--use-mpi`` (OMPI_COMM_WORLD_*), explicit flags, or torchrun's environment."""
    env = os.environ
    if getattr(args, "use_mpi", False) and "OMPI_COMM_WORLD_SIZE" in env:
        args.world_size = int(env["OMPI_COMM_WORLD_SIZE"])
        args.rank = int(env["OMPI_COMM_WORLD_RANK"])
        args.local_rank = int(env["OMPI_COMM_WORLD_LOCAL_RANK"])
        return
    if args.world_size is None:
        args.world_size = int(env.get("WORLD_SIZE", 1))
    if args.rank is None:
        args.rank = int(env.get("RANK", 0))
    if args.local_rank is None:
        args.local_rank = int(env.get("LOCAL_RANK", args.rank))


def parse_comma_delimited_arg(arg: str, cast_fn: Callable[[str], object]) -> List[object]:
    return [cast_fn(x) for x in str(arg).split(",")]


def model_choices():
    return list(MODEL_CONFIGS.keys())


def device_memory_gb(default: float = 180.0) -> float:
    try:
        import torch
        if torch.cuda.is_available():
            return torch.cuda.get_device_properties(0).total_memory / 2 ** 30
    except Exception:
        pass
    return default
