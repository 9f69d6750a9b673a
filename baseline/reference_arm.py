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


class _Grads(list):
    """What ``torch.autograd.grad`` returns to the reference in this process: a list, because the
    driver concatenates ``[dy] + all_grads[n:]`` (test_transformer_terapipe.py:156-166), which
    also adds to a tuple from the left, because the reference's recompute function returns
    ``(None, None) + grads`` (checkpoint.py:43).  Torch of the reference's era returned a tuple
    and its driver code predates the list concatenation failing; both call shapes must work."""

    def __radd__(self, other):
        if isinstance(other, tuple):
            return other + tuple(self)
        return list(other) + list(self)


def _autograd_grad_returns_list(torch) -> None:
    """See :class:`_Grads`.  In this process only, wrap ``torch.autograd.grad``."""
    original = torch.autograd.grad
    if getattr(original, "_returns_list", False):
        return

    def grad(*args, **kwargs):
        return _Grads(original(*args, **kwargs))

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


class ReferenceArm:
    """The unmodified reference behind the block interface of bench.py: ``setup`` (imports and
    process group), ``measure`` (one model / layout / slice schedule through the reference's own
    ``NCCLTransformerRunner.step``), ``tp_block`` and ``finish``."""
    name = "reference"

    def __init__(self, args, timed_steps, ClockSampler, slices_for, config_dict, l2_note):
        self.args = args
        self.timed_steps, self.ClockSampler = timed_steps, ClockSampler
        self.slices_for, self.config_dict, self.l2_note = slices_for, config_dict, l2_note

    def setup(self, rank, world, local):
        """Returns None when ready, else the reason the reference cannot run here."""
        self.rank, self.world, self.local = rank, world, local
        if not os.path.isfile(os.path.join(REF, "test_transformer_terapipe.py")):
            return "baseline/_ref is missing: the reference has not been installed"
        # the reference's modules (mpu, utils, transformer_models, ...) must win over anything else
        for p in (os.path.join(HERE, "apex_stub"), REF):
            sys.path.insert(0, p)
        for name in ("mpu", "utils", "transformer_models", "checkpoint", "memory_model"):
            sys.modules.pop(name, None)
        try:
            import torch
            import torch.distributed as dist
            if not torch.cuda.is_available():
                return "no CUDA device"
            torch.cuda.set_device(local)
            self.device = torch.device("cuda", local)
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            os.environ.setdefault("RANK", str(rank))
            os.environ.setdefault("WORLD_SIZE", str(world))
            with contextlib.redirect_stdout(sys.stderr):
                dist.init_process_group("nccl", device_id=self.device)
                import test_transformer_terapipe as ref
                ref.np = _NumpyCompat(ref.np)
                _autograd_grad_returns_list(torch)
                _cat_out_across_devices(torch)
                assert os.path.dirname(os.path.abspath(ref.__file__)) == REF
            self.ref = ref
        except Exception as e:  # noqa: BLE001
            return f"reference set-up failed: {type(e).__name__}: {str(e)[:200]}"
        return None

    def measure(self, spec, steps, warmup, main=False, **_):
        import gc
        import torch
        with contextlib.redirect_stdout(sys.stderr):
            from transformer_models import MODEL_CONFIGS, TransformerConfig
            import mpu as ref_mpu
            tp, pp = spec["tp"], spec["pp"]
            dp = self.world // (tp * pp)
            config = TransformerConfig.from_predefined_model(spec["model"], n_devices=self.world,
                                                             batch_size=spec["batch"])
            if spec.get("n_layers") is not None:
                config.n_layers = spec["n_layers"]
            seq_len = MODEL_CONFIGS[spec["model"]][2]
            batch_slices, seq_slices = self.slices_for(spec, seq_len, self.args if main else None)
            recompute = bool(spec.get("checkpoint_gradients", False))
            torch.cuda.reset_peak_memory_stats()
            runner = self.ref.NCCLTransformerRunner(
                config, batch_slices, seq_slices, "env://", self.world, dp, tp, pp, self.rank,
                self.local, mixed_precision=True, use_mpi=False, init_process_group=False,
                checkpoint_gradients=recompute)
            for _ in range(warmup):
                runner.step()
            sampler = self.ClockSampler(self.local)
            if self.rank == 0:
                sampler.start()
            ms = self.timed_steps(runner.step, steps, self.world, self.device)
            clocks = sampler.stop() if self.rank == 0 else None
            peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30
            del runner
            ref_mpu.destroy_model_parallel()
            gc.collect()
            torch.cuda.empty_cache()
        ms_per_step = ms / steps
        tokens = spec["batch"] * seq_len * dp
        value = tokens / (ms_per_step / 1e3)
        return {
            "value": value, "unit": "tokens/s", "tokens_per_s": value, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "iteration_latency_s": ms_per_step / 1e3,
            "data": "synthetic N(0,1) hidden states created on the device by the reference's own "
                    "step(), random-init weights",
            "config": self.config_dict(
                model=spec["model"], n_layers=config.n_layers, hidden=config.embedding_dim,
                heads=config.num_attention_heads, global_batch=tokens // seq_len, seq_len=seq_len,
                parallelism=f"pp{pp}xtp{tp}xdp{dp}", batch_slices=batch_slices, seq_slices=seq_slices,
                activation="relu", mixed_precision="fp32 master weights, loss scale 128",
                optimizer="torch.optim.Adam(fused=True) standing in for apex FusedAdam",
                attention_recompute=recompute, cuda_graph=False, launch_plan=False,
                tp_comm="nccl" if tp > 1 else "none", dp_comm="nccl" if dp > 1 else "none",
                l2=self.l2_note),
            "gpu_launches": None, "clocks": clocks,
            "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms_per_step,
                    "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "the reference's public step() draws its inputs on the device and reads "
                            "nothing back; this repeats the device-timed number"},
            "peak_memory_gb_torch_allocator": round(peak_gb, 2),
        }

    def tp_block(self, spec, steps, warmup):
        block = self.measure(spec, steps, warmup)
        return {"config": block["config"], "steps": steps, "warmup": warmup,
                "modes": {"nccl": {"ms_per_step": block["ms_per_step"], "tokens_per_s": block["value"],
                                   "clocks": block["clocks"]}}}

    def finish(self):
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
