"""Activation recompute that composes with ``torch.autograd.grad``.

``CheckpointFunction.apply(fn, n_tensor_args, *args)`` runs ``fn(*args[:n])`` without
recording a graph and replays it in backward; ``args[n:]`` are parameters that ``fn``
closes over and that must receive gradients.  Same calling contract as the reference's
checkpoint.py (:24-43).  Unlike ``torch.utils.checkpoint`` it works when the caller
differentiates with ``torch.autograd.grad`` (which the token-slice backward does).
"""
from __future__ import annotations

import warnings

import torch


def detach_variable(inputs):
    if not isinstance(inputs, tuple):
        raise RuntimeError(f"only a tuple of tensors is supported, got {type(inputs).__name__}")
    return tuple(t.detach().requires_grad_(t.requires_grad) for t in inputs)


def check_backward_validity(inputs):
    if not any(t.requires_grad for t in inputs):
        warnings.warn("None of the inputs have requires_grad=True. Gradients will be None")


class CheckpointFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_function, length, *args):
        ctx.run_function = run_function
        ctx.n_tensor_args = length
        ctx.stash = args
        with torch.no_grad():
            return run_function(*args[:length])

    @staticmethod
    def backward(ctx, *output_grads):
        n = ctx.n_tensor_args
        replay_inputs = list(detach_variable(tuple(ctx.stash[:n])))
        params = list(ctx.stash[n:])
        with torch.enable_grad():
            outputs = ctx.run_function(*replay_inputs)
        if isinstance(outputs, torch.Tensor):
            outputs = (outputs,)
        wanted = [t for t in replay_inputs + params if t.requires_grad]
        grads = iter(torch.autograd.grad(outputs, wanted, output_grads, allow_unused=True))
        full = [next(grads) if t.requires_grad else None for t in replay_inputs + params]
        return (None, None) + tuple(full)
