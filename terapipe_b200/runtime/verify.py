"""Cross-configuration golden check (``--verify save|load``).

``save`` (one rank, no slicing) runs one step and writes into ``path``

    input.pt          the ``[seq, batch, hidden]`` input
    model.ckpt        the full, unsharded state dict, keys ``layers.layers.<global layer>.<param>``
    model.grad.ckpt   the same keys -> parameter gradients

``load`` (any TP x PP x slicing) reads them under file locks, shards weights and reference
gradients for this rank with :func:`slice_state_dict`, runs one step and compares every
parameter gradient.  File names, key layout and sharding rules are those of the reference's
verifier (terapipe.py:318-423); unlike it, a tolerance suited to the compute dtype is used
instead of ``allclose`` defaults, and the result is returned as well as asserted.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..models import TransformerConfig, slice_state_dict
from ..utils import uniform_slice

try:  # serialises readers/writers that share a directory
    from filelock import FileLock
except Exception:  # pragma: no cover - filelock is an optional dependency
    import contextlib

    def FileLock(path):  # noqa: N802
        return contextlib.nullcontext()


def _build(engine: str, cfg, batch_slices, seq_slices, device, dtype):
    if engine == "b200":
        from .engine import StageEngine
        return StageEngine(cfg, batch_slices, seq_slices, dtype=dtype or torch.float16,
                           init="reference", use_graph=False)
    from .portable import PortablePipeline
    return PortablePipeline(cfg, batch_slices, seq_slices, device=device,
                            mixed_precision=dtype is not None, dtype=dtype or torch.float16)


def _grads(runner, engine, x):
    if engine == "b200":
        if runner.is_first:
            runner.set_input(x)
        runner.compute_grads()
        return runner.named_grads(), runner.state_dict()
    runner.compute_grads(x if runner.is_first else None)
    return runner.named_grads(), runner.state_dict()


def verify_one_step(path: str, mode: str, model: str = "test", n_layers: Optional[int] = None,
                    batch_size: int = 1, tp: int = 1, pp: int = 1, n_batch_slices: int = 1,
                    n_input_slices: int = 1, device: str = "cpu", engine: str = "portable",
                    dtype=None, atol: Optional[float] = None, rtol: Optional[float] = None,
                    activation: str = "gelu"):
    os.makedirs(path, exist_ok=True)
    world = dist.get_world_size() if dist.is_initialized() else 1
    if not mpu.model_parallel_is_initialized() and dist.is_initialized():
        mpu.initialize_model_parallel(tp, pp, verbose=False)
    cfg = TransformerConfig.from_predefined_model(model, n_devices=world, batch_size=batch_size,
                                                  n_layers=n_layers, activation=activation)
    files = {k: os.path.join(path, k) for k in ("input.pt", "model.ckpt", "model.grad.ckpt")}
    if mode == "save":
        if not (world == 1 and tp == 1 and pp == 1 and n_batch_slices == 1 and n_input_slices == 1):
            raise AssertionError("save runs on one rank without slicing")
        runner = _build(engine, cfg, [batch_size], [cfg.seq_len], device, dtype)
        g = torch.Generator().manual_seed(4321)
        x = torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g)
        grads, state = _grads(runner, engine, x.to(device))
        for name, obj in (("input.pt", x), ("model.ckpt", state), ("model.grad.ckpt", grads)):
            with FileLock(files[name] + ".lock"):
                torch.save(obj if name == "input.pt" else {k: v.cpu() for k, v in obj.items()},
                           files[name])
        return {"ok": True, "saved": sorted(files)}
    if mode != "load":
        raise ValueError("mode must be 'save' or 'load'")
    loaded = {}
    for name in files:
        with FileLock(files[name] + ".lock"):
            loaded[name] = torch.load(files[name], map_location="cpu")
    topo = mpu.get_topology()
    rank = dist.get_rank() if dist.is_initialized() else 0
    _, pp_rank, tp_rank = topo.coords(rank)
    runner = _build(engine, cfg, uniform_slice(batch_size, n_batch_slices),
                    uniform_slice(cfg.seq_len, n_input_slices), device, dtype)
    weights = slice_state_dict(cfg.n_layers, loaded["model.ckpt"], topo.tp, tp_rank, topo.pp, pp_rank)
    want = slice_state_dict(cfg.n_layers, loaded["model.grad.ckpt"], topo.tp, tp_rank, topo.pp, pp_rank)
    runner.load_state_dict(weights)
    got, _ = _grads(runner, engine, loaded["input.pt"].to(device))
    low_precision = dtype is not None or engine == "b200"
    atol = atol if atol is not None else (2e-3 if low_precision else 1e-5)
    rtol = rtol if rtol is not None else (5e-2 if low_precision else 1e-4)
    worst, bad = 0.0, []
    for k, ref in want.items():
        mine = got[k].detach().float().cpu()
        err = (mine - ref.float()).abs().max().item()
        worst = max(worst, err)
        if low_precision:
            rel = (mine - ref.float()).norm() / (ref.float().norm() + 1e-12)
            if rel > rtol:
                bad.append((k, float(rel)))
        elif not torch.allclose(mine, ref.float(), atol=atol, rtol=rtol):
            bad.append((k, err))
    assert not bad, f"rank {rank}: gradients differ from the saved run: {bad[:4]}"
    return {"ok": True, "max_abs_err": worst, "n_params": len(want)}
