"""Region mappings between replicated and tensor-parallel activations.

Four autograd functions with conjugate forward/backward collectives, the NCCL-backed
form of the reference's mpu/mappings.py:79-144:

========  ================  ================
mapping   forward           backward
========  ================  ================
copy      identity          all-reduce
reduce    all-reduce        identity
scatter   keep my chunk     all-gather
gather    all-gather        keep my chunk
========  ================  ================

All bypass communication when the tensor-parallel size is 1.  On B200 the production
engine replaces the "linear followed by reduce" pair by one fused GEMM + all-reduce
kernel over NVLink peer memory (terapipe_b200/ops); these torch.distributed versions are
the portable path (CPU/gloo tests) and the oracle for the fused kernels.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .initialize import (get_model_parallel_group, get_model_parallel_rank,
                         get_model_parallel_world_size)
from .utils import split_tensor_along_last_dim


def _reduce(x: torch.Tensor) -> torch.Tensor:
    if get_model_parallel_world_size() == 1:
        return x
    dist.all_reduce(x, group=get_model_parallel_group())
    return x


def _split(x: torch.Tensor) -> torch.Tensor:
    tp = get_model_parallel_world_size()
    if tp == 1:
        return x
    return split_tensor_along_last_dim(x, tp)[get_model_parallel_rank()].contiguous()


def _gather(x: torch.Tensor) -> torch.Tensor:
    tp = get_model_parallel_world_size()
    if tp == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(tp)]
    parts[get_model_parallel_rank()] = x
    dist.all_gather(parts, x.contiguous(), group=get_model_parallel_group())
    return torch.cat(parts, dim=x.dim() - 1).contiguous()


def _make(name, fwd, bwd):
    def forward(ctx, x):
        return fwd(x)

    def backward(ctx, g):
        return bwd(g)

    return type(name, (torch.autograd.Function,),
                {"forward": staticmethod(forward), "backward": staticmethod(backward)})


def _ident(x):
    return x


_CopyToModelParallelRegion = _make("_CopyToModelParallelRegion", _ident,
                                   lambda g: _reduce(g.contiguous().clone()))
_ReduceFromModelParallelRegion = _make("_ReduceFromModelParallelRegion",
                                       lambda x: _reduce(x.contiguous().clone()), _ident)
_ScatterToModelParallelRegion = _make("_ScatterToModelParallelRegion", _split, _gather)
_GatherFromModelParallelRegion = _make("_GatherFromModelParallelRegion", _gather, _split)


def copy_to_model_parallel_region(x):
    return _CopyToModelParallelRegion.apply(x)


def reduce_from_model_parallel_region(x):
    return _ReduceFromModelParallelRegion.apply(x)


def scatter_to_model_parallel_region(x):
    return _ScatterToModelParallelRegion.apply(x)


def gather_from_model_parallel_region(x):
    return _GatherFromModelParallelRegion.apply(x)
