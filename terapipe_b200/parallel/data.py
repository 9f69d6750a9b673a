"""Broadcast a dict of tensors from the first rank of a tensor-parallel group.

Counterpart of the reference's mpu/data.py (:23-116): one broadcast carries the shapes
(up to 4 dims per key), a second carries the flattened payload.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch
import torch.distributed as dist

from .initialize import (get_model_parallel_group, get_model_parallel_rank,
                         get_model_parallel_src_rank)

_MAX_DATA_DIM = 4


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if (
        torch.cuda.is_available() and dist.get_backend() == "nccl") else torch.device("cpu")


def _check_data_types(keys, data, target_dtype):
    for k in keys:
        if data[k].dtype != target_dtype:
            raise AssertionError(f"{k} has dtype {data[k].dtype}, expected {target_dtype}")


def _build_key_size_numel_dictionaries(keys: Sequence[str], data):
    sizes = [0] * (_MAX_DATA_DIM * len(keys))
    if get_model_parallel_rank() == 0:
        for i, k in enumerate(keys):
            shape = tuple(data[k].shape)
            if len(shape) > _MAX_DATA_DIM:
                raise AssertionError("too many dimensions to broadcast")
            sizes[i * _MAX_DATA_DIM:i * _MAX_DATA_DIM + len(shape)] = shape
    packed = torch.tensor(sizes, dtype=torch.long, device=_device())
    dist.broadcast(packed, get_model_parallel_src_rank(), group=get_model_parallel_group())
    packed = packed.cpu().tolist()
    key_size, key_numel, total = {}, {}, 0
    for i, k in enumerate(keys):
        shape = [s for s in packed[i * _MAX_DATA_DIM:(i + 1) * _MAX_DATA_DIM] if s > 0]
        numel = 1
        for s in shape:
            numel *= s
        key_size[k], key_numel[k] = shape, numel
        total += numel
    return key_size, key_numel, total


def broadcast_data(keys: Sequence[str], data: Dict[str, torch.Tensor], datatype):
    """Every rank of the group gets the tensors that tensor-parallel rank 0 holds."""
    key_size, key_numel, total = _build_key_size_numel_dictionaries(keys, data)
    if get_model_parallel_rank() == 0:
        _check_data_types(keys, data, datatype)
        flat = torch.cat([data[k].contiguous().view(-1) for k in keys]).to(_device())
    else:
        flat = torch.empty(total, dtype=datatype, device=_device())
    dist.broadcast(flat, get_model_parallel_src_rank(), group=get_model_parallel_group())
    out, offset = {}, 0
    for k in keys:
        out[k] = flat.narrow(0, offset, key_numel[k]).view(key_size[k])
        offset += key_numel[k]
    return out
