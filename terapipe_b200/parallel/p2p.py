"""Shard-to-shard pipeline links.

Tensor-parallel rank *i* of a stage exchanges token slices with tensor-parallel rank *i*
of the neighbouring stage through point-to-point send/recv (NCCL on GPUs, gloo on CPU).
The reference instead broadcasts inside 2-rank groups from the last TP rank of a stage
to the first TP rank of the next and then fans out inside the TP group
(terapipe.py:98-151); the data every rank ends up holding is the same.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import initialize as _init


def send_forward(y: torch.Tensor) -> None:
    nxt = _init.get_pipeline_next_rank()
    if nxt is not None:
        dist.send(y.contiguous(), nxt)


def recv_forward(buf: torch.Tensor) -> torch.Tensor:
    prv = _init.get_pipeline_prev_rank()
    if prv is not None:
        dist.recv(buf, prv)
    return buf


def send_backward(dx: torch.Tensor) -> None:
    prv = _init.get_pipeline_prev_rank()
    if prv is not None:
        dist.send(dx.contiguous(), prv)


def recv_backward(buf: torch.Tensor) -> torch.Tensor:
    nxt = _init.get_pipeline_next_rank()
    if nxt is not None:
        dist.recv(buf, nxt)
    return buf


class PipelineSendOperator(torch.autograd.Function):
    """Differentiable send to the next stage: forward sends ``x``, backward receives the
    gradient of ``x`` from there (the role of terapipe.py:98-124 in the reference)."""

    @staticmethod
    def forward(ctx, x):
        send_forward(x.detach())
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        if _init.get_pipeline_next_rank() is None:
            return grad
        buf = torch.empty_like(grad)
        recv_backward(buf)
        return buf


class PipelineRecvOperator(torch.autograd.Function):
    """Differentiable receive from the previous stage: forward fills ``x`` with the received
    slice, backward sends the gradient back (terapipe.py:127-151)."""

    @staticmethod
    def forward(ctx, x):
        if _init.get_pipeline_prev_rank() is None:
            return x.view_as(x)
        buf = torch.empty_like(x)
        recv_forward(buf)
        return buf

    @staticmethod
    def backward(ctx, grad):
        send_backward(grad)
        return grad


pipeline_send = PipelineSendOperator.apply
pipeline_recv = PipelineRecvOperator.apply
