"""Training checkpoints: one shard file per rank, written atomically, re-shardable.

The reference has no resumable training state (only the verification snapshot, terapipe.py:
368-423).  A shard holds, for the layers and tensor-parallel slice of its rank, the fp32 master
weights and Adam moments in the state-dict key layout ``layers.layers.<local layer>.<param>``,
plus the step count, Adam bias-correction state, loss scale, the layout it was written with and
the host RNG state.  ``reshard`` converts a complete set of shards to another TP x PP layout
with the same slicing rules as ``slice_state_dict``.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..models.slicing import merge_state_dicts, slice_state_dict

FORMAT_VERSION = 1


def shard_path(directory: str, pp_rank: int, tp_rank: int, dp_rank: int = 0) -> str:
    return os.path.join(directory, f"shard_pp{pp_rank}_tp{tp_rank}_dp{dp_rank}.pt")


def _named(engine, buf) -> Dict[str, torch.Tensor]:
    from .engine import PARAM_ORDER
    # `get_param` gives the model's own shapes (an engine that pads heads for its kernels keeps
    # the padding to itself), so a checkpoint does not depend on the engine's internal layout
    return {f"layers.layers.{l}.{name}": engine.get_param(l, name, buf).detach().float().cpu().clone()
            for l in range(engine.n_layers) for name in PARAM_ORDER}


def _atomic_save(obj, path: str) -> None:
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _gather_sharded_state(engine) -> None:
    """With the fused data-parallel update (``dp_comm="fused"``) a rank keeps master weights and
    Adam moments up to date only for the chunk of the flat parameter space it owns.  Before a
    save every replica fetches the other chunks from their owners, so that each replica's
    buffers are complete again (collective over the data-parallel group)."""
    import torch.distributed as dist
    from .. import parallel as mpu
    if getattr(engine, "dp_sym", None) is None:
        return
    group = mpu.get_data_parallel_group()
    for buf in (engine.master, engine.exp_avg, engine.exp_avg_sq):
        own = torch.zeros_like(buf)
        for _, _, b, e in engine._dp_ranges:
            own[b:e] = buf[b:e]
        dist.all_reduce(own, group=group)      # every element has exactly one owner
        buf.copy_(own)


def save_checkpoint(engine, directory: str) -> str:
    """Write this rank's shard.  Call it on every rank, between steps: with the fused
    data-parallel update the replicas first exchange the chunks of master weights and moments
    they own (a collective), and the ranks of a tensor- or data-parallel group meet at a host
    barrier afterwards, so that no rank runs ahead into a device-side wait while another is
    still writing its file."""
    import torch.distributed as dist
    os.makedirs(directory, exist_ok=True)
    _gather_sharded_state(engine)
    blob = {
        "version": FORMAT_VERSION,
        "layout": {"tp": engine.tp, "pp": engine.pp, "dp": engine.dp, "tp_rank": engine.tp_idx,
                   "pp_rank": engine.pp_idx, "dp_rank": engine.dp_idx,
                   "n_layers": engine.cfg.n_layers},
        "step": engine.step_count, "loss_scale": engine.loss_scale,
        "adam_state": engine.adam_state.detach().cpu().clone(),
        "master": _named(engine, engine.master), "exp_avg": _named(engine, engine.exp_avg),
        "exp_avg_sq": _named(engine, engine.exp_avg_sq),
        "rng": {"torch": torch.get_rng_state()},
    }
    path = shard_path(directory, engine.pp_idx, engine.tp_idx, engine.dp_idx)
    _atomic_save(blob, path)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    return path


def load_checkpoint(engine, directory: str) -> dict:
    """Restore this rank's shard written with the SAME layout; returns the shard's metadata.
    Every data-parallel replica reads the shard of replica 0 (complete, see save_checkpoint)."""
    import torch.distributed as dist
    from .engine import PARAM_ORDER
    path = shard_path(directory, engine.pp_idx, engine.tp_idx, 0)
    blob = torch.load(path, map_location="cpu")
    lay = blob["layout"]
    if (lay["tp"], lay["pp"]) != (engine.tp, engine.pp):
        raise ValueError(f"checkpoint layout tp{lay['tp']}xpp{lay['pp']} differs from the engine's "
                         f"tp{engine.tp}xpp{engine.pp}; run reshard() first")
    if lay["n_layers"] != engine.cfg.n_layers:
        raise ValueError(f"checkpoint holds {lay['n_layers']} layers, the engine {engine.cfg.n_layers}")
    if float(blob.get("loss_scale", engine.loss_scale)) != float(engine.loss_scale):
        raise ValueError(f"checkpoint was written with loss scale {blob['loss_scale']}, the engine "
                         f"uses {engine.loss_scale}")
    for key, buf in (("master", engine.master), ("exp_avg", engine.exp_avg),
                     ("exp_avg_sq", engine.exp_avg_sq)):
        for l in range(engine.n_layers):
            for name in PARAM_ORDER:
                engine.set_param(l, name, blob[key][f"layers.layers.{l}.{name}"], buf)
    engine.model.copy_(engine.master)
    engine.adam_state.copy_(blob["adam_state"])
    engine.step_count = blob["step"]
    torch.set_rng_state(blob["rng"]["torch"])
    if dist.is_available() and dist.is_initialized():
        torch.cuda.synchronize()
        dist.barrier()
    return {"step": blob["step"], "layout": lay}


def reshard(src_dir: str, dst_dir: str, tp: int, pp: int) -> None:
    """Rewrite a complete checkpoint for another tensor/pipeline layout (host only)."""
    first = torch.load(shard_path(src_dir, 0, 0), map_location="cpu")
    lay = first["layout"]
    n_layers = lay["n_layers"]
    shards = {(s, r): torch.load(shard_path(src_dir, s, r), map_location="cpu")
              for s in range(lay["pp"]) for r in range(lay["tp"])}
    os.makedirs(dst_dir, exist_ok=True)
    full = {key: merge_state_dicts(n_layers, {k: v[key] for k, v in shards.items()},
                                   lay["tp"], lay["pp"])
            for key in ("master", "exp_avg", "exp_avg_sq")}
    for s in range(pp):
        for r in range(tp):
            blob = dict(first)
            blob["layout"] = dict(lay, tp=tp, pp=pp, tp_rank=r, pp_rank=s, dp_rank=0)
            for key in full:
                blob[key] = slice_state_dict(n_layers, full[key], tp, r, pp, s)
            _atomic_save(blob, shard_path(dst_dir, s, r))
