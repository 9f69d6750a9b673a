"""Experiment runner with the constructor and methods of the reference's
``NCCLTransformerRunner`` (test_transformer_terapipe.py:29-352), on top of this package's
engines: the sm_100a :class:`StageEngine` on a GPU, the portable autograd pipeline otherwise.
"""
from __future__ import annotations

import time
from typing import Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..models import TransformerConfig
from ..utils import set_random_seed, timeout

LOSS_SCALE_FACTOR = 128.0


def init_distributed(init_method: str, world_size: int, rank: int, local_rank: int,
                     backend: Optional[str] = None) -> str:
    """Initialise torch.distributed (NCCL when CUDA is present, else gloo) and warm the
    communicator up with one tiny all-reduce, as the reference does at start-up."""
    use_cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if use_cuda else "gloo")
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        kwargs = {"device_id": torch.device("cuda", local_rank)} if backend == "nccl" else {}
        dist.init_process_group(backend=backend, init_method=init_method, world_size=world_size,
                                rank=rank, **kwargs)
    probe = torch.zeros(1, device="cuda" if backend == "nccl" else "cpu")
    dist.all_reduce(probe)
    return backend


class NCCLTransformerRunner:
    def __init__(self, config: TransformerConfig, batch_slices: Sequence[int],
                 seq_slices: Sequence[int], distributed_init_method: str, world_size: int,
                 data_parallel_size: int, model_parallel_size: int, pipeline_parallel_size: int,
                 rank: int, local_rank: int, mixed_precision: bool = False, use_mpi: bool = False,
                 init_process_group: bool = False, checkpoint_gradients: bool = False,
                 engine: str = "auto", dtype=torch.float16, tp_comm: str = "fused",
                 use_graph=None, init: str = "device"):
        self.config = config
        self.batch_slices, self.seq_slices = list(batch_slices), list(seq_slices)
        self.rank, self.local_rank, self.world_size = rank, local_rank, world_size
        self.data_parallel_size = data_parallel_size
        self.model_parallel_size = model_parallel_size
        self.pipeline_parallel_size = pipeline_parallel_size
        self.mixed_precision = mixed_precision
        self.checkpoint_gradients = checkpoint_gradients
        if init_process_group or (world_size > 1 and not dist.is_initialized()):
            init_distributed(distributed_init_method, world_size, rank, local_rank)
        if dist.is_initialized():
            mpu.destroy_model_parallel()
            mpu.initialize_model_parallel(model_parallel_size, pipeline_parallel_size, verbose=rank == 0)
        elif torch.cuda.is_available():
            torch.cuda.set_device(local_rank)
        set_random_seed(0)
        if dist.is_initialized():
            mpu.model_parallel_cuda_manual_seed(0)
        use_b200 = engine == "b200" or (engine == "auto" and torch.cuda.is_available()
                                        and mixed_precision
                                        and config.attention_heads_dim <= 128
                                        and config.attention_heads_dim % 8 == 0)
        self.engine_kind = "b200" if use_b200 else "portable"
        if use_b200:
            from .engine import StageEngine
            self.impl = StageEngine(config, self.batch_slices, self.seq_slices, dtype=dtype,
                                    loss_scale=LOSS_SCALE_FACTOR, init=init, use_graph=use_graph,
                                    tp_comm=tp_comm)
        else:
            from .portable import PortablePipeline
            self.impl = PortablePipeline(config, self.batch_slices, self.seq_slices,
                                         mixed_precision=mixed_precision,
                                         checkpoint_gradients=checkpoint_gradients, dtype=dtype)
        self._step = 0

    @property
    def n_batch_slices(self):
        return len(self.batch_slices)

    @property
    def n_input_slices(self):
        return len(self.seq_slices)

    def _input(self):
        impl = self.impl
        if not impl.is_first:
            return None
        c = self.config
        seed = 977 + 7919 * impl.dp_idx + self._step
        if torch.cuda.is_available() and self.engine_kind == "b200":
            # drawn on the device, as the reference does (test_transformer_terapipe.py:181-189):
            # the timed step must not contain host random-number generation or a pageable copy
            g = torch.Generator(device=impl.device).manual_seed(seed)
            return torch.randn(c.seq_len, c.batch_size, c.embedding_dim, generator=g,
                               device=impl.device, dtype=impl.dtype)
        g = torch.Generator().manual_seed(seed)
        return torch.randn(c.seq_len, c.batch_size, c.embedding_dim, generator=g)

    def step(self):
        x = self._input()
        if self.engine_kind == "b200":
            if x is not None:
                self.impl.set_input(x)
            self.impl.step()
        else:
            self.impl.step(None if x is None else x.to(self.impl.device, self.impl.low_dtype))
        self._step += 1

    @timeout(seconds=500)
    def run(self, n_steps, warmup_steps=5, verbose=True):
        """Times ``n_steps`` iterations.  Returns (mean, std) of the wall-clock step time in
        seconds over the steps after the warm-up, as the reference does
        (test_transformer_terapipe.py:289-303).  Also recorded, for the drivers' extended result
        rows: ``last_device_ms`` (mean step time between CUDA events on the launching stream;
        wall clock on CPU) and ``last_peak_memory_gb``."""
        times, dev_ms = [], []
        cuda = torch.cuda.is_available()
        if cuda:
            torch.cuda.reset_peak_memory_stats()
        for _ in range(n_steps):
            t0 = time.time()
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            self.step()
            if cuda:
                e1.record()
                torch.cuda.synchronize()
                dev_ms.append(e0.elapsed_time(e1))
            times.append(time.time() - t0)
            if not cuda:
                dev_ms.append(times[-1] * 1e3)
            if verbose:
                print("rank", self.rank, "step_time:", times[-1], flush=True)
        skip = warmup_steps if len(times) > warmup_steps else 0
        kept = times[skip:]
        mean, std = float(np.mean(kept)), float(np.std(kept))
        self.last_device_ms = float(np.mean(dev_ms[skip:]))
        self.last_peak_memory_gb = torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else 0.0
        if skip:
            print("rank", self.rank, "step_time_mean:", mean, "step_time_std:", std, flush=True)
        return mean, std

    def max_over_ranks_device_ms(self):
        """``last_device_ms`` of the slowest rank (the job's step time)."""
        value = getattr(self, "last_device_ms", None)
        if value is None or not dist.is_initialized() or dist.get_world_size() == 1:
            return value
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
        t = torch.tensor([value], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def _grads_for(self, batch_slices, seq_slices, x):
        if self.engine_kind == "b200":
            from .engine import StageEngine
            eng = StageEngine(self.config, batch_slices, seq_slices, dtype=self.impl.dtype,
                              init="device", use_graph=False, tp_comm="nccl")
            eng.load_state_dict(self.impl.state_dict())
            if eng.is_first:
                eng.set_input(x)
            eng.compute_grads()
            return eng.named_grads()
        from .portable import PortablePipeline
        p = PortablePipeline(self.config, batch_slices, seq_slices,
                             mixed_precision=self.mixed_precision,
                             checkpoint_gradients=self.checkpoint_gradients)
        p.load_state_dict(self.impl.state_dict())
        p.compute_grads(None if x is None else x.to(p.device, p.low_dtype))
        return p.named_grads()

    def verify(self, rtol=None):
        """Gradients of the sliced schedule against the unsliced one on the same input and
        weights; prints the mean absolute difference per parameter and asserts a tolerance."""
        x = self._input()
        sliced = self._grads_for(self.batch_slices, self.seq_slices, x)
        whole = self._grads_for([sum(self.batch_slices)], [sum(self.seq_slices)], x)
        rtol = rtol if rtol is not None else (5e-2 if self.mixed_precision else 1e-4)
        worst = 0.0
        for k in sliced:
            diff = (sliced[k].float() - whole[k].float())
            print(diff.abs().mean().item(), tuple(sliced[k].shape))
            rel = (diff.norm() / (whole[k].float().norm() + 1e-12)).item()
            worst = max(worst, rel)
        assert worst < rtol, f"sliced and unsliced gradients differ: relative error {worst}"
        return worst


# The reference splits the runner into a base class (model, schedule, optimizer) and a subclass
# that adds step/run/verify; here one class does both and the base name is kept as an alias.
NCCLTransformer = NCCLTransformerRunner
