"""Cross entropy over vocabulary-sharded logits.

Counterpart of the reference's mpu/cross_entropy.py (:25-110).  Three small collectives
over the tensor-parallel group per call: max, the target logit (owned by exactly one
rank) and the sum of exponentials.  Backward is ``softmax - onehot`` on the local shard.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .initialize import (get_model_parallel_group, get_model_parallel_rank,
                         get_model_parallel_world_size)
from .utils import VocabUtility


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target):
        group, tp = get_model_parallel_group(), get_model_parallel_world_size()
        logits = logits.float()
        row_max = logits.max(dim=-1)[0]
        if tp > 1:
            dist.all_reduce(row_max, op=dist.ReduceOp.MAX, group=group)
        shifted = logits - row_max.unsqueeze(-1)
        first, last = VocabUtility.vocab_range_from_per_partition_vocab_size(
            logits.size(-1), get_model_parallel_rank(), tp)
        outside = (target < first) | (target >= last)
        local_target = (target - first).masked_fill(outside, 0)
        picked = shifted.gather(-1, local_target.unsqueeze(-1)).squeeze(-1)
        picked = picked.masked_fill(outside, 0.0)
        exp = shifted.exp()
        denom = exp.sum(dim=-1)
        if tp > 1:
            dist.all_reduce(picked, group=group)
            dist.all_reduce(denom, group=group)
        loss = denom.log() - picked
        ctx.save_for_backward(exp / denom.unsqueeze(-1), outside, local_target)
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        softmax, outside, local_target = ctx.saved_tensors
        grad = softmax.clone()
        onehot = (~outside).to(grad.dtype).unsqueeze(-1)
        grad.scatter_add_(-1, local_target.unsqueeze(-1), -onehot)
        return grad * grad_out.unsqueeze(-1), None


def vocab_parallel_cross_entropy(vocab_parallel_logits, target):
    return _VocabParallelCrossEntropy.apply(vocab_parallel_logits, target)
