"""Reference arm of bench.py: the unmodified reference, installed under ``baseline/_ref``,
driven through its own ``NCCLTransformerRunner.step`` (test_transformer_terapipe.py:270-287).

Only the harness around it is ours: process-group initialisation from torchrun's
environment (the runner is then built with ``init_process_group=False``, the path the
reference's own sweep takes for every experiment after the first), CUDA-event timing around
``step()`` with the maximum taken over ranks, and an ``apex.optimizers.FusedAdam`` stand-in
(apex is not installed on this image).  None of this repository's models, kernels or engine
is imported on this path.
"""
from __future__ import annotations

import contextlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


class _NumpyCompat:
    """numpy as the reference's driver sees it.  With numpy >= 2 and current torch,
    ``np.array(tuple_of_cuda_tensors, dtype='O')`` (test_transformer_terapipe.py:204) tries to
    convert every tensor to an ndarray and raises; numpy of the reference's era built a 1-D
    object array holding the tensors.  This proxy restores that behaviour for that one call
    shape and forwards everything else to numpy untouched."""

    def __init__(self, np_module):
        self._np = np_module

    def __getattr__(self, name):
        return getattr(self._np, name)

    def array(self, obj, *args, **kwargs):
        dtype = kwargs.get("dtype", args[0] if args else None)
        if dtype in ("O", object) and isinstance(obj, (tuple, list)):
            out = self._np.empty(len(obj), dtype=object)
            for i, item in enumerate(obj):
                out[i] = item
            return out
        return self._np.array(obj, *args, **kwargs)


def _autograd_grad_returns_list(torch) -> None:
    """The reference's backward loop concatenates ``[dy] + all_grads[n:]``
    (test_transformer_terapipe.py:156-166), which needs ``torch.autograd.grad`` to hand back a
    list; current torch returns a tuple.  In this process only, wrap it to return a list."""
    original = torch.autograd.grad
    if getattr(original, "_returns_list", False):
        return

    def grad(*args, **kwargs):
        return list(original(*args, **kwargs))

    grad._returns_list = True
    torch.autograd.grad = grad


def _cat_out_across_devices(torch) -> None:
    """With tensor parallelism the reference builds the full master weight on the CPU and does
    ``torch.cat(chunks, dim, out=weight)`` with ``weight`` on the GPU (mpu/layers.py:65-79);
    current torch refuses an ``out`` on another device.  In this process only, perform the
    concatenation where the chunks live and copy the result into ``out``."""
    original = torch.cat
    if getattr(original, "_cross_device_out", False):
        return

    def cat(tensors, dim=0, *, out=None):
        if out is not None and len(tensors) and tensors[0].device != out.device:
            out.copy_(original(list(tensors), dim))
            return out
        return original(tensors, dim) if out is None else original(tensors, dim, out=out)

    cat._cross_device_out = True
    torch.cat = cat


def _unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run(args, dist_env, timed_steps, ClockSampler, slices_from_args) -> None:
    rank, world, local = dist_env()
    if not os.path.isfile(os.path.join(REF, "test_transformer_terapipe.py")):
        if rank == 0:
            _unavailable("baseline/_ref is missing: the reference has not been installed")
        return
    # the reference's modules (mpu, utils, transformer_models, ...) must win over anything else
    for p in (os.path.join(HERE, "apex_stub"), REF):
        sys.path.insert(0, p)
    for name in ("mpu", "utils", "transformer_models", "checkpoint", "memory_model"):
        sys.modules.pop(name, None)
    try:
        import torch
        import torch.distributed as dist
        if not torch.cuda.is_available():
            if rank == 0:
                _unavailable("no CUDA device")
            return
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        os.environ.setdefault("RANK", str(rank))
        os.environ.setdefault("WORLD_SIZE", str(world))
        with contextlib.redirect_stdout(sys.stderr):
            dist.init_process_group("nccl", device_id=device)
            import test_transformer_terapipe as ref
            ref.np = _NumpyCompat(ref.np)
            _autograd_grad_returns_list(torch)
            _cat_out_across_devices(torch)
            from transformer_models import MODEL_CONFIGS, TransformerConfig
            assert os.path.dirname(os.path.abspath(ref.__file__)) == REF
            pp = args.pp if args.pp is not None else world // args.tp
            dp = world // (args.tp * pp)
            config = TransformerConfig.from_predefined_model(args.model, n_devices=world,
                                                             batch_size=args.batch)
            if args.n_layers is not None:
                config.n_layers = args.n_layers
            seq_len = MODEL_CONFIGS[args.model][2]

            from utils import uniform_slice
            if args.schedule:
                with open(args.schedule) as f:
                    sched = json.load(f)
                if isinstance(sched, list):
                    sched = sched[getattr(args, "schedule_index", 0)]
                batch_slices, seq_slices = list(sched["batch_slices"]), list(sched["input_slices"])
            else:
                batch_slices = uniform_slice(args.batch, args.batch_slices)
                seq_slices = uniform_slice(seq_len, args.seq_slices)
            runner = ref.NCCLTransformerRunner(
                config, batch_slices, seq_slices, "env://", world, dp, args.tp, pp, rank, local,
                mixed_precision=True, use_mpi=False, init_process_group=False,
                checkpoint_gradients=False)
            warmup = max(args.warmup, 3)
            for _ in range(warmup):
                runner.step()
            sampler = ClockSampler(local)
            if rank == 0:
                sampler.start()
            ms = timed_steps(runner.step, args.steps, world, device)
            clocks = sampler.stop() if rank == 0 else None
        ms_per_step = ms / args.steps
        tokens = args.batch * seq_len * dp
        if rank == 0:
            value = tokens / (ms_per_step / 1e3)
            print(json.dumps({
                "metric": "training throughput (tokens/s), GPT-3-shaped decoder, fwd+bwd+Adam per iteration",
                "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": ms_per_step, "iteration_latency_s": ms_per_step / 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "fp16", "data": "synthetic N(0,1) hidden states created on the device by the reference's own step(), random-init weights",
                "impl": "reference",
                "config": {"model": args.model, "n_layers": config.n_layers,
                           "global_batch": tokens // seq_len, "seq_len": seq_len,
                           "parallelism": f"pp{pp}xtp{args.tp}xdp{dp}", "batch_slices": batch_slices,
                           "seq_slices": seq_slices, "activation": "relu (the reference's layer)",
                           "optimizer": "torch.optim.Adam(fused=True) standing in for apex FusedAdam",
                           "l2": "per-step working set far exceeds the 126 MB L2"},
                "gpu_launches": None, "clocks": clocks,
                "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0,
                        "note": "the reference's public step() draws its inputs on the device and reads nothing back; this repeats the device-timed number"},
            }), flush=True)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        if rank == 0:
            _unavailable(f"reference run failed: {type(e).__name__}: {str(e)[:200]}")
