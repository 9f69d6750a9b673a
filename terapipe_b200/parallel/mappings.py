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

Sequence-parallel regions (tokens, dim 0, sharded over the tensor-parallel group between the
GEMM pairs; the layout the fused all-gather->GEMM / GEMM->reduce-scatter kernels work on):

===============  ======================  ======================
mapping          forward                 backward
===============  ======================  ======================
seq scatter      keep my token chunk     all-gather (tokens)
seq gather       all-gather (tokens)     reduce-scatter (tokens), or keep my chunk when the
                                         consumer is replicated
seq reduce-scat  reduce-scatter (tokens) all-gather (tokens)
===============  ======================  ======================

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


def _split_tokens(x: torch.Tensor) -> torch.Tensor:
    tp = get_model_parallel_world_size()
    if tp == 1:
        return x
    if x.size(0) % tp:
        raise ValueError(f"{x.size(0)} tokens cannot be split over {tp} tensor-parallel ranks")
    return x.chunk(tp, dim=0)[get_model_parallel_rank()].contiguous()


def _gather_tokens(x: torch.Tensor) -> torch.Tensor:
    tp = get_model_parallel_world_size()
    if tp == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(tp)]
    dist.all_gather(parts, x.contiguous(), group=get_model_parallel_group())
    return torch.cat(parts, dim=0)


def _reduce_scatter_tokens(x: torch.Tensor) -> torch.Tensor:
    tp = get_model_parallel_world_size()
    if tp == 1:
        return x
    if x.size(0) % tp:
        raise ValueError(f"{x.size(0)} tokens cannot be split over {tp} tensor-parallel ranks")
    chunks = [c.contiguous() for c in x.chunk(tp, dim=0)]
    out = torch.empty_like(chunks[0])
    if dist.get_backend(get_model_parallel_group()) == "gloo":
        # gloo has no reduce-scatter: sum everything, keep my chunk
        full = x.contiguous().clone()
        dist.all_reduce(full, group=get_model_parallel_group())
        return full.chunk(tp, dim=0)[get_model_parallel_rank()].contiguous()
    dist.reduce_scatter(out, chunks, group=get_model_parallel_group())
    return out


_ScatterToSequenceParallelRegion = _make("_ScatterToSequenceParallelRegion", _split_tokens, _gather_tokens)
_GatherFromSequenceParallelRegion = _make("_GatherFromSequenceParallelRegion", _gather_tokens,
                                          _reduce_scatter_tokens)
_ReduceScatterToSequenceParallelRegion = _make("_ReduceScatterToSequenceParallelRegion",
                                               _reduce_scatter_tokens, _gather_tokens)
_GatherSequenceToReplicatedRegion = _make("_GatherSequenceToReplicatedRegion", _gather_tokens,
                                          _split_tokens)


def scatter_to_sequence_parallel_region(x):
    return _ScatterToSequenceParallelRegion.apply(x)


def gather_from_sequence_parallel_region(x, tensor_parallel_output_grad=True):
    """All-gather the token chunks.  When the consumer is tensor parallel (every rank produces a
    different gradient of the gathered tensor) the backward is a reduce-scatter; when it is
    replicated (every rank computes the same thing, e.g. a loss) the backward keeps this rank's
    chunk."""
    if tensor_parallel_output_grad:
        return _GatherFromSequenceParallelRegion.apply(x)
    return _GatherSequenceToReplicatedRegion.apply(x)


def reduce_scatter_to_sequence_parallel_region(x):
    return _ReduceScatterToSequenceParallelRegion.apply(x)


def copy_to_model_parallel_region(x):
    return _CopyToModelParallelRegion.apply(x)


def reduce_from_model_parallel_region(x):
    return _ReduceFromModelParallelRegion.apply(x)


def scatter_to_model_parallel_region(x):
    return _ScatterToModelParallelRegion.apply(x)


def gather_from_model_parallel_region(x):
    return _GatherFromModelParallelRegion.apply(x)
