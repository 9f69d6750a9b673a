#!/usr/bin/env python
"""Module-style driver: one model/parallel setting, scalar flags, iteration timing, and the
cross-configuration golden check ``--verify save|load --verify-path DIR``
(flags of the reference's terapipe.py:427-444, plus ``--n-layers`` and ``--tp-comm``).

``TeraPipe`` wraps a stage's layers as an ``nn.Module`` whose forward runs the token-slice
schedule and whose output can be back-propagated with ``.backward()``.
"""
import argparse

import numpy as np
import torch
import torch.distributed as dist
from torch import nn

from terapipe_b200 import parallel as mpu
from terapipe_b200.models import MODEL_CONFIGS, TransformerConfig, slice_state_dict  # noqa: F401
from terapipe_b200.parallel.p2p import (PipelineRecvOperator, PipelineSendOperator,  # noqa: F401
                                        pipeline_recv, pipeline_send)
from terapipe_b200.runtime import cli, verify
from terapipe_b200.runtime.portable import PortablePipeline, TransformerLayers  # noqa: F401
from terapipe_b200.runtime.runner import NCCLTransformerRunner, init_distributed
from terapipe_b200.utils import uniform_slice


LOSS_SCALE_FACTOR = 128.0


def loss_func(y):
    """Training loss of the drivers: the mean of all output elements (terapipe.py:48-49)."""
    return torch.mean(y)


def initialize_distributed_env(distributed_init_method, rank, local_rank, world_size,
                               model_parallel_size, pipeline_parallel_size):
    init_distributed(distributed_init_method, world_size, rank, local_rank)
    mpu.initialize_model_parallel(model_parallel_size, pipeline_parallel_size)
    torch.manual_seed(0)
    mpu.model_parallel_cuda_manual_seed(0)


class _PipelineFunction(torch.autograd.Function):
    """Forward = token-slice forward of the stage; backward = reverse-order slice replay that
    accumulates parameter gradients and returns the input gradient."""

    @staticmethod
    def forward(ctx, module, x, anchor):
        pipe = module.pipeline
        with torch.enable_grad():
            ctx.rec = pipe.forward_step(x.detach() if pipe.is_first else None)
        ctx.pipe = pipe
        outs = [torch.cat([ctx.rec[bi, si][1].detach() for si in range(len(pipe.seq_slices))], 0)
                for bi in range(len(pipe.batch_slices))]
        return torch.cat(outs, dim=1)

    @staticmethod
    def backward(ctx, grad_y):
        pipe = ctx.pipe
        pipe.backward_step(ctx.rec, output_grad=grad_y if pipe.is_last else None)
        for p, g in zip(pipe.params, pipe.main_grads):
            p.grad = g.to(p.dtype) if p.grad is None else p.grad + g.to(p.dtype)
            g.zero_()
        return None, None, None


class TeraPipe(nn.Module):
    """``TeraPipe(config, batch_slices, seq_slices)(x)``: the stage's output ``[L, B, H]`` (a
    dummy of the same shape on stages that are not last).  State-dict keys are
    ``layers.layers.<local layer>.<param>``."""

    def __init__(self, config, batch_slices, seq_slices, mixed_precision=False, device=None):
        super().__init__()
        self.pipeline = PortablePipeline(config, batch_slices, seq_slices,
                                         mixed_precision=mixed_precision, device=device)
        self.layers = self.pipeline.layers

    def forward(self, inputs=None):
        if inputs is None:
            c = self.pipeline.config
            inputs = torch.zeros(c.seq_len, c.batch_size, c.embedding_dim)
        # `anchor` ties the output to the autograd graph even when the input needs no gradient
        return _PipelineFunction.apply(self, inputs, self.pipeline.params[0])


class TeraPipeBackwardPassHook(torch.autograd.Function):
    """Identity on ``y`` whose backward replays the token slices in reverse order
    (reference API, terapipe.py:154-214).  For user-written sliced forwards:

    * ``outputs[i, j]`` is the output of batch slice ``i``, token slice ``j`` (attached to its
      own autograd graph);
    * ``cache_inputs[i, j]`` are the detached, grad-requiring cache tensors that slice ``j``
      read, ``cache_outputs[i, j]`` the cache tensors it produced for slice ``j + 1``.

    Backward walks ``j`` from last to first: slice ``j`` is differentiated with the gradient of
    its output plus the cache gradients that slice ``j + 1`` left in ``cache_inputs[i, j + 1]``."""

    @staticmethod
    def forward(ctx, y, outputs, cache_inputs, cache_outputs, batch_slices, seq_slices, batch_dim,
                sequence_dim, cat_outputs):
        ctx.state = (outputs, cache_inputs, cache_outputs, list(batch_slices), list(seq_slices),
                     batch_dim, sequence_dim, cat_outputs)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        from terapipe_b200.models import grid_slice_batch_and_sequence
        outputs, cache_in, cache_out, batch_slices, seq_slices, bdim, sdim, cat = ctx.state
        ctx.state = None
        nb, ns = len(batch_slices), len(seq_slices)
        grads = (grid_slice_batch_and_sequence(grad_y, batch_slices=batch_slices, seq_slices=seq_slices,
                                               batch_dim=bdim, sequence_dim=sdim, requires_grad=False)
                 if cat else None)
        for i in reversed(range(nb)):
            from_next = []
            for j in reversed(range(ns)):
                dy = grads[i, j] if cat else torch.empty_like(outputs[i, j])
                produced = list(cache_out[i, j]) if j < ns - 1 else []
                torch.autograd.backward([outputs[i, j]] + produced, [dy] + from_next)
                from_next = [t.grad for t in cache_in[i, j]]
        return (None,) * 9


def terapipe_backward_hook(outputs, cache_inputs, cache_outputs, batch_slices, seq_slices,
                           batch_dim=1, sequence_dim=0, cat_outputs=False):
    """Tensor whose ``backward()`` drives :class:`TeraPipeBackwardPassHook`: the concatenated
    slice outputs when ``cat_outputs`` (take a loss of it), otherwise a scalar placeholder (for
    stages whose slice gradients arrive through their own receive operators)."""
    with torch.no_grad():
        if cat_outputs:
            y = torch.cat([torch.cat(list(row), dim=sequence_dim) for row in outputs], dim=batch_dim)
        else:
            y = torch.tensor(0.0)
    y.requires_grad_()
    return TeraPipeBackwardPassHook.apply(y, outputs, cache_inputs, cache_outputs, batch_slices,
                                          seq_slices, batch_dim, sequence_dim, cat_outputs)


def initialize_model(args):
    """(config, layers, pipelined_layers) of this rank's stage from driver arguments
    (terapipe.py:274-288); ``config.n_layers`` is the stage's share of ``n_total_layers``."""
    config = TransformerConfig.from_predefined_model(args.model, n_devices=getattr(args, "world_size", 1),
                                                     batch_size=args.batch_size,
                                                     n_layers=getattr(args, "n_layers", None))
    pipelined_layers = TeraPipe(config, uniform_slice(config.batch_size, args.n_batch_slices),
                                uniform_slice(config.seq_len, args.n_input_slices),
                                mixed_precision=getattr(args, "mixed_precision", False))
    config.n_total_layers = config.n_layers
    config.n_layers = len(mpu.get_topology().layers_of_stage(
        config.n_total_layers, mpu.get_pipeline_parallel_group_rank()))
    return config, pipelined_layers.layers, pipelined_layers


def verify_one_step(args):
    """``--verify save|load`` of the drivers (terapipe.py:368-423): write, or check against, the
    files ``input.pt``, ``model.ckpt`` and ``model.grad.ckpt`` in ``args.verify_path``."""
    use_b200 = torch.cuda.is_available() and getattr(args, "mixed_precision", False)
    return verify.verify_one_step(
        args.verify_path, args.verify, model=args.model, n_layers=getattr(args, "n_layers", None),
        batch_size=args.batch_size, tp=args.model_parallel_size, pp=args.pipeline_parallel_size,
        n_batch_slices=args.n_batch_slices, n_input_slices=args.n_input_slices,
        device="cuda" if torch.cuda.is_available() else "cpu",
        engine="b200" if use_b200 else "portable")


def measure_iteration_time(args, n_warmup_steps=2):
    config = TransformerConfig.from_predefined_model(args.model, n_devices=args.world_size,
                                                     batch_size=args.batch_size,
                                                     n_layers=args.n_layers)
    dp = args.world_size // (args.model_parallel_size * args.pipeline_parallel_size)
    runner = NCCLTransformerRunner(
        config, uniform_slice(args.batch_size, args.n_batch_slices),
        uniform_slice(config.seq_len, args.n_input_slices),
        f"tcp://{args.ip_address}:{args.port}", args.world_size, dp, args.model_parallel_size,
        args.pipeline_parallel_size, args.rank, args.local_rank,
        mixed_precision=args.mixed_precision, init_process_group=args.world_size > 1,
        tp_comm=args.tp_comm)
    mean, std = runner.run(args.n_steps + n_warmup_steps, warmup_steps=n_warmup_steps, verbose=False)
    return mean, std


def main():
    parser = argparse.ArgumentParser(description="token-level pipeline parallel training step")
    cli.add_rank_arguments(parser)
    parser.add_argument("--model-parallel-size", type=int, default=1)
    parser.add_argument("--pipeline-parallel-size", type=int, default=1)
    parser.add_argument("--model", type=str, default="test", choices=cli.model_choices())
    parser.add_argument("--n-layers", type=int, default=None)
    parser.add_argument("--batch-size", type=int, default=1)
    parser.add_argument("--n-batch-slices", type=int, default=1)
    parser.add_argument("--n-input-slices", type=int, default=1)
    parser.add_argument("--n-steps", type=int, default=10)
    parser.add_argument("--mixed-precision", action="store_true", default=False)
    parser.add_argument("--verify", type=str, default=None, choices=["save", "load"])
    parser.add_argument("--verify-path", type=str, default="verify_data")
    parser.add_argument("--tp-comm", default="fused", choices=["nccl", "fused", "sp"])
    args = parser.parse_args()
    cli.resolve_ranks(args)
    if args.verify:
        if args.world_size > 1 or torch.cuda.is_available():
            init_distributed(f"tcp://{args.ip_address}:{args.port}", args.world_size, args.rank,
                             args.local_rank)
        out = verify_one_step(args)
        print("rank", args.rank, "verify", args.verify, out, flush=True)
    else:
        mean, std = measure_iteration_time(args)
        print("rank", args.rank, "step_time_mean:", mean, "step_time_std:", std, flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
