"""Small arithmetic helpers of the tensor-parallel layer (reference: mpu/utils.py:20-70)."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch


def ensure_divisibility(numerator: int, denominator: int) -> None:
    if numerator % denominator != 0:
        raise AssertionError(f"{numerator} is not divisible by {denominator}")


def divide(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def split_tensor_along_last_dim(tensor: torch.Tensor, num_partitions: int,
                                contiguous_split_chunks: bool = False) -> Sequence[torch.Tensor]:
    width = divide(tensor.size(-1), num_partitions)
    parts = torch.split(tensor, width, dim=tensor.dim() - 1)
    return tuple(p.contiguous() for p in parts) if contiguous_split_chunks else parts


class VocabUtility:
    """Half-open vocabulary range ``[first, last)`` owned by one tensor-parallel rank."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition: int, rank: int,
                                                  world_size: int) -> Tuple[int, int]:
        first = rank * per_partition
        return first, first + per_partition

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab: int, rank: int,
                                           world_size: int) -> Tuple[int, int]:
        return VocabUtility.vocab_range_from_per_partition_vocab_size(
            divide(global_vocab, world_size), rank, world_size)
