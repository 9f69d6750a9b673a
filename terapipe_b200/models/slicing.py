"""Cutting activations into (batch slice, token slice) grids, layers into stages, and
full state dicts into (stage, tensor-parallel rank) shards.

References: grid slicing transformer_models.py:393-409; layer split terapipe.py:276-279;
state-dict shards terapipe.py:318-365.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Sequence

import numpy as np
import torch

from ..parallel.topology import Topology


def grid_slice_batch_and_sequence(x, batch_slices: Sequence[int], seq_slices: Sequence[int],
                                  requires_grad=False, batch_dim=1, sequence_dim=0):
    """Object ndarray ``[len(batch_slices), len(seq_slices)]`` of contiguous, detached
    blocks of ``x``.  Slice arguments are lists of lengths that must sum to the sizes."""
    if sum(seq_slices) != x.size(sequence_dim) or sum(batch_slices) != x.size(batch_dim):
        raise AssertionError("slice lengths must add up to the tensor's sizes")
    grid = np.empty((len(batch_slices), len(seq_slices)), dtype=object)
    b0 = 0
    for i, nb in enumerate(batch_slices):
        s0 = 0
        for j, ns in enumerate(seq_slices):
            block = x.narrow(sequence_dim, s0, ns).narrow(batch_dim, b0, nb)
            grid[i, j] = block.detach().clone(memory_format=torch.contiguous_format) \
                .requires_grad_(requires_grad)
            s0 += ns
        b0 += nb
    return grid


def uniform_slice_x(x, n_slices: int) -> List[torch.Tensor]:
    from ..utils import uniform_slice
    out, start = [], 0
    for n in uniform_slice(x.size(0), n_slices):
        out.append(x[start:start + n])
        start += n
    return out


def uniform_slice_layers(transformer_layers, n_devices=None):
    n_devices = n_devices or max(torch.cuda.device_count(), 1)
    topo = Topology(n_devices, 1, n_devices)
    return [[transformer_layers[i] for i in topo.layers_of_stage(len(transformer_layers), s)]
            for s in range(n_devices)]


_ROW_SHARDED = ("attn.in_proj.weight", "attn.in_proj.bias", "fc1.weight", "fc1.bias")
_COL_SHARDED = ("attn.out_proj.weight", "fc2.weight")


def slice_state_dict(n_layers: int, full_state: Dict[str, torch.Tensor], tp: int, tp_rank: int,
                     pp: int, pp_rank: int, prefix: str = "layers.layers.") -> "OrderedDict":
    """Shard a full (unsharded, all layers) state dict for one (stage, TP rank).

    Keys are ``<prefix><global layer>.<param>`` and are renumbered to local layer ids.
    ``in_proj`` and ``fc1`` weights/biases are cut into contiguous row blocks (which, with
    the per-head interleaved q,k,v column order, are contiguous head groups);
    ``out_proj`` and ``fc2`` weights into contiguous column blocks; everything else is
    replicated."""
    layer_ids = Topology(tp * pp, tp, pp).layers_of_stage(n_layers, pp_rank)
    first = layer_ids.start
    out = OrderedDict()
    for key, value in full_state.items():
        if not key.startswith(prefix):
            continue
        layer_str, name = key[len(prefix):].split(".", 1)
        gid = int(layer_str)
        if gid not in layer_ids:
            continue
        if name in _ROW_SHARDED:
            n = value.size(0) // tp
            value = value.narrow(0, tp_rank * n, n)
        elif name in _COL_SHARDED:
            n = value.size(1) // tp
            value = value.narrow(1, tp_rank * n, n)
        out[f"{prefix}{gid - first}.{name}"] = value.clone()
    return out


def merge_state_dicts(n_layers: int, shards: Dict[tuple, Dict[str, torch.Tensor]], tp: int,
                      pp: int, prefix: str = "layers.layers.") -> "OrderedDict":
    """Inverse of :func:`slice_state_dict`: ``shards[(pp_rank, tp_rank)]`` -> full dict."""
    topo = Topology(tp * pp, tp, pp)
    out = OrderedDict()
    for s in range(pp):
        first = topo.layers_of_stage(n_layers, s).start
        for key in shards[(s, 0)]:
            layer_str, name = key[len(prefix):].split(".", 1)
            parts = [shards[(s, r)][key] for r in range(tp)]
            if name in _ROW_SHARDED:
                value = torch.cat(parts, dim=0)
            elif name in _COL_SHARDED:
                value = torch.cat(parts, dim=1)
            else:
                value = parts[0].clone()
            out[f"{prefix}{int(layer_str) + first}.{name}"] = value
    return out


def save_layers_and_inputs(layers, grad_layers, layer_ids, inputs, prefix):
    """Legacy per-layer files: ``prefix.<i>``, ``prefix.grad.<i>``, ``prefix.inputs``."""
    for i, layer, grad in zip(layer_ids, layers, grad_layers):
        torch.save(layer.state_dict(), f"{prefix}.{i}")
        torch.save(grad, f"{prefix}.grad.{i}")
    torch.save(inputs, f"{prefix}.inputs")


def load_layers(layers, layer_ids, prefix):
    for i, layer in zip(layer_ids, layers):
        layer.load_state_dict(torch.load(f"{prefix}.{i}"))


def load_grads(layer_ids, prefix):
    return [torch.load(f"{prefix}.grad.{i}") for i in layer_ids]


def load_inputs(prefix):
    return torch.load(f"{prefix}.inputs")
