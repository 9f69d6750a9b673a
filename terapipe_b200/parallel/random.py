"""Per-region CUDA RNG streams and an RNG-replaying activation checkpoint.

Counterpart of the reference's mpu/random.py (:32-243).  Two generator states exist per
rank: the *default* state (same inside a tensor-parallel group, used in replicated
regions) and a named ``model-parallel-rng`` state (``seed + 2718 + tp_rank``, used
inside sharded regions) so that e.g. dropout differs between shards but matches between
data-parallel replicas.  On a machine without CUDA the tracker keeps CPU generator
states instead, which lets the bookkeeping be tested anywhere.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

from .initialize import get_data_parallel_rank, get_model_parallel_rank

_MODEL_PARALLEL_RNG_TRACKER_NAME = "model-parallel-rng"


def _cuda_ok() -> bool:
    return torch.cuda.is_available()


def _get_state():
    return torch.cuda.get_rng_state() if _cuda_ok() else torch.get_rng_state()


def _set_cuda_rng_state(new_state, device=-1):
    """Install a generator state without the device synchronisation of a full reseed."""
    if not _cuda_ok():
        torch.set_rng_state(new_state)
        return
    idx = torch.cuda.current_device() if device == -1 else torch.device("cuda", device).index
    torch.cuda.default_generators[idx].set_state(new_state)


def _seed(seed: int):
    if _cuda_ok():
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)


class CudaRNGStatesTracker:
    """Named generator states that can be forked into and restored from."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.states_ = {}
        self.seeds_ = set()

    def get_states(self):
        return dict(self.states_)

    def set_states(self, states):
        self.states_ = states

    def add(self, name, seed):
        if seed in self.seeds_:
            raise Exception(f"seed {seed} already exists")
        if name in self.states_:
            raise Exception(f"cuda rng state {name} already exists")
        self.seeds_.add(seed)
        saved = _get_state()
        _seed(seed)
        self.states_[name] = _get_state()
        _set_cuda_rng_state(saved)

    @contextlib.contextmanager
    def fork(self, name=_MODEL_PARALLEL_RNG_TRACKER_NAME):
        if name not in self.states_:
            raise Exception(f"cuda rng state {name} is not added")
        saved = _get_state()
        _set_cuda_rng_state(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = _get_state()
            _set_cuda_rng_state(saved)


_TRACKER = CudaRNGStatesTracker()


def get_cuda_rng_tracker() -> CudaRNGStatesTracker:
    return _TRACKER


def model_parallel_cuda_manual_seed(seed: int, verbose: bool = False) -> None:
    """Seed the default state with ``seed`` and the model-parallel state with
    ``seed + 2718 + tp_rank``.  Call after ``initialize_model_parallel``."""
    mp_seed = seed + 2718 + get_model_parallel_rank()
    if verbose and dist.is_initialized() and dist.get_rank() == 0:
        print(f"> cuda seeds: tp rank {get_model_parallel_rank()} dp rank "
              f"{get_data_parallel_rank()} model-parallel {mp_seed} data-parallel {seed}",
              flush=True)
    _TRACKER.reset()
    _seed(seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG_TRACKER_NAME, mp_seed)


class CheckpointFunction(torch.autograd.Function):
    """Recompute-in-backward that replays the CPU, CUDA and tracker RNG states, so a
    segment containing dropout regenerates the same masks."""

    @staticmethod
    def forward(ctx, run_function, *args):
        ctx.run_function = run_function
        ctx.cpu_state = torch.get_rng_state()
        ctx.dev_state = _get_state()
        ctx.tracker_states = _TRACKER.get_states()
        with torch.no_grad():
            out = run_function(*args)
        ctx.save_for_backward(*args)
        return out

    @staticmethod
    def backward(ctx, *grads):
        if not torch.autograd._is_checkpoint_valid():
            raise RuntimeError("checkpointing is not compatible with .grad(); use .backward()")
        inputs = tuple(t.detach().requires_grad_(t.requires_grad) for t in ctx.saved_tensors)
        keep = (torch.get_rng_state(), _get_state(), _TRACKER.get_states())
        torch.set_rng_state(ctx.cpu_state)
        _set_cuda_rng_state(ctx.dev_state)
        _TRACKER.set_states(ctx.tracker_states)
        with torch.enable_grad():
            out = ctx.run_function(*inputs)
        torch.set_rng_state(keep[0])
        _set_cuda_rng_state(keep[1])
        _TRACKER.set_states(keep[2])
        if isinstance(out, torch.Tensor):
            out = (out,)
        torch.autograd.backward(out, grads)
        return (None,) + tuple(t.grad for t in inputs)


def checkpoint(function, *args):
    return CheckpointFunction.apply(function, *args)
