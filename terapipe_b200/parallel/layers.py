"""Tensor-parallel linear and embedding modules (portable torch path).

API of the reference's mpu/layers.py (:85-353).  Weights are drawn as the FULL master
matrix from the global CPU generator on every rank and then sliced, so a weight is the
same whatever the tensor-parallel size (mpu/layers.py:41-82); biases start at zero.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn
from torch.nn import init

from .initialize import get_model_parallel_rank, get_model_parallel_world_size
from .mappings import (copy_to_model_parallel_region, gather_from_model_parallel_region,
                       gather_from_sequence_parallel_region, reduce_from_model_parallel_region,
                       reduce_scatter_to_sequence_parallel_region, scatter_to_model_parallel_region)
from .utils import VocabUtility, divide


def _initialize_affine_weight(weight, output_size, input_size, per_partition_size,
                              partition_dim, init_method, stride=1,
                              initialize_locally=False, return_master_weight=False):
    """Fill ``weight`` with my tensor-parallel shard of an ``[output, input]`` master."""
    if initialize_locally and return_master_weight:
        raise AssertionError("a locally initialised weight has no master weight")
    weight.model_parallel = True
    weight.partition_dim = partition_dim
    weight.stride = stride
    tp = get_model_parallel_world_size()
    if tp == 1 or initialize_locally:
        with torch.no_grad():
            local = torch.empty(weight.shape, dtype=torch.float32)
            init_method(local)
            weight.copy_(local)
        return weight if return_master_weight else None
    master = torch.empty(output_size, input_size, dtype=torch.float32)
    init_method(master)
    chunk = divide(per_partition_size, stride)
    pieces = torch.split(master, chunk, dim=partition_dim)[get_model_parallel_rank()::tp]
    with torch.no_grad():
        weight.copy_(torch.cat(pieces, dim=partition_dim))
    return master.to(weight.dtype) if return_master_weight else None


class VocabParallelEmbedding(nn.Module):
    """Embedding table sharded over the vocabulary; rows outside my range contribute
    zeros and an all-reduce assembles the result."""

    def __init__(self, num_embeddings, embedding_dim, init_method=init.xavier_normal_):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.vocab_start_index, self.vocab_end_index = \
            VocabUtility.vocab_range_from_global_vocab_size(
                num_embeddings, get_model_parallel_rank(), get_model_parallel_world_size())
        self.num_embeddings_per_partition = self.vocab_end_index - self.vocab_start_index
        self.weight = nn.Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim))
        _initialize_affine_weight(self.weight, num_embeddings, embedding_dim,
                                  self.num_embeddings_per_partition, 0, init_method)

    def forward(self, ids):
        outside = (ids < self.vocab_start_index) | (ids >= self.vocab_end_index)
        local_ids = (ids - self.vocab_start_index).masked_fill(outside, 0)
        out = F.embedding(local_ids, self.weight)
        out = out.masked_fill(outside.unsqueeze(-1), 0.0)
        return reduce_from_model_parallel_region(out)


class ParallelEmbedding(nn.Module):
    """Embedding table sharded over the embedding dimension; outputs are all-gathered."""

    def __init__(self, num_embeddings, embedding_dim, init_method=init.xavier_normal_,
                 keep_master_weight_for_test=False):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        tp = get_model_parallel_world_size()
        self.embedding_dim_per_partition = divide(embedding_dim, tp)
        self.weight = nn.Parameter(torch.empty(num_embeddings, self.embedding_dim_per_partition))
        self.master_weight = _initialize_affine_weight(
            self.weight, num_embeddings, embedding_dim, self.embedding_dim_per_partition, 1,
            init_method, return_master_weight=keep_master_weight_for_test)

    def forward(self, ids):
        ids = copy_to_model_parallel_region(ids) if ids.is_floating_point() else ids
        return gather_from_model_parallel_region(F.embedding(ids, self.weight))


class ColumnParallelLinear(nn.Module):
    """``Y = X W^T + b`` with W ``[out, in]`` sharded by rows (output features):
    local weight ``[out/tp, in]``, bias ``[out/tp]``."""

    def __init__(self, input_size, output_size, bias=True, gather_output=True,
                 init_method=init.xavier_normal_, stride=1, initialize_locally=False,
                 keep_master_weight_for_test=False, device="cpu", sequence_parallel=False):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.gather_output = gather_output
        # sequence_parallel: the input holds this rank's chunk of the tokens (dim 0); it is
        # all-gathered before the product (backward: reduce-scatter of the input gradient)
        self.sequence_parallel = sequence_parallel
        tp = get_model_parallel_world_size()
        self.output_size_per_partition = divide(output_size, tp)
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, input_size))
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition))
            self.bias.model_parallel = True
            self.bias.partition_dim = 0
            self.bias.stride = stride
        else:
            self.register_parameter("bias", None)
        self.master_weight = _initialize_affine_weight(
            self.weight, output_size, input_size, self.output_size_per_partition, 0,
            init_method, stride=stride, initialize_locally=initialize_locally,
            return_master_weight=keep_master_weight_for_test)
        self.to(device)

    def forward(self, x):
        x = gather_from_sequence_parallel_region(x) if self.sequence_parallel \
            else copy_to_model_parallel_region(x)
        y = F.linear(x, self.weight, self.bias)
        return gather_from_model_parallel_region(y) if self.gather_output else y


class RowParallelLinear(nn.Module):
    """``Y = X W^T + b`` with W ``[out, in]`` sharded by columns (input features):
    local weight ``[out, in/tp]``; partial products are all-reduced, then the
    (unsharded) bias is added."""

    def __init__(self, input_size, output_size, bias=True, input_is_parallel=False,
                 init_method=init.xavier_normal_, stride=1, initialize_locally=False,
                 keep_master_weight_for_test=False, device="cpu", sequence_parallel=False):
        super().__init__()
        self.input_size, self.output_size = input_size, output_size
        self.input_is_parallel = input_is_parallel
        # sequence_parallel: partial products are reduce-scattered over the tokens (dim 0)
        # instead of all-reduced; the output is this rank's token chunk
        self.sequence_parallel = sequence_parallel
        tp = get_model_parallel_world_size()
        self.input_size_per_partition = divide(input_size, tp)
        self.weight = nn.Parameter(torch.empty(output_size, self.input_size_per_partition))
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size))
        else:
            self.register_parameter("bias", None)
        self.master_weight = _initialize_affine_weight(
            self.weight, output_size, input_size, self.input_size_per_partition, 1,
            init_method, stride=stride, initialize_locally=initialize_locally,
            return_master_weight=keep_master_weight_for_test)
        self.to(device)

    def forward(self, x, return_reduce_time=False):
        if not self.input_is_parallel:
            x = scatter_to_model_parallel_region(x)
        partial = F.linear(x, self.weight)
        if return_reduce_time:
            # Debug timing of the collective alone: drain the device and line the ranks up
            # on both sides (reference: mpu/layers.py:336-345).
            if partial.is_cuda:
                torch.cuda.synchronize()
            dist.barrier()
            t0 = time.time()
        y = reduce_scatter_to_sequence_parallel_region(partial) if self.sequence_parallel \
            else reduce_from_model_parallel_region(partial)
        if return_reduce_time:
            if partial.is_cuda:
                torch.cuda.synchronize()
            dist.barrier()
            elapsed = time.time() - t0
        if self.bias is not None:
            y = y + self.bias
        return (y, elapsed) if return_reduce_time else y
