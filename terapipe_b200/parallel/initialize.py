"""Process-group state for tensor / pipeline / data parallelism.

Same accessor surface as the reference's ``mpu/initialize.py`` (:108-236), built on
the arithmetic in :mod:`terapipe_b200.parallel.topology`.  Pipeline links are
shard-to-shard: tensor-parallel rank *i* of stage *k* talks to tensor-parallel rank *i*
of stage *k+1*, so every rank (not just the first/last of its TP group) owns a
predecessor and a successor link.  ``torch.distributed.new_group`` is collective over
the world, so every rank creates every group in the same order.
"""
from __future__ import annotations

from typing import Optional

import torch.distributed as dist

from .topology import Topology

_STATE = None


class _State:
    def __init__(self, topo: Topology, rank: int):
        self.topo = topo
        self.rank = rank
        self.dp_idx, self.pp_idx, self.tp_idx = topo.coords(rank)
        self.dp_group = None
        self.tp_group = None
        self.pp_group = None
        self.pred_group = None   # group in which I am the sender of the forward pass
        self.succ_group = None   # group in which I am the receiver of the forward pass


def initialize_model_parallel(model_parallel_size: int, pipeline_parallel_size: int = 1,
                              verbose: bool = True) -> Topology:
    """Create DP, TP, per-shard pipeline and adjacent-stage groups.

    Example with 16 ranks, tp=4, pp=2: stages [0..3] -> [4..7] form replica 0 and
    [8..11] -> [12..15] replica 1; DP groups are {0,8}, {1,9}, ...
    """
    global _STATE
    assert dist.is_initialized(), "torch.distributed must be initialised first"
    topo = Topology(dist.get_world_size(), model_parallel_size, pipeline_parallel_size)
    rank = dist.get_rank()
    if verbose and rank == 0:
        print(f"> tensor parallel {topo.tp} x pipeline {topo.pp} x data {topo.dp}", flush=True)
    st = _State(topo, rank)
    for ranks in topo.dp_groups():
        g = dist.new_group(ranks)
        if rank in ranks:
            st.dp_group = g
    for ranks in topo.tp_groups():
        g = dist.new_group(ranks)
        if rank in ranks:
            st.tp_group = g
    if topo.pp > 1:
        for ranks in topo.pp_groups():
            g = dist.new_group(ranks)
            if rank in ranks:
                st.pp_group = g
        for pred, succ in topo.stage_pairs():
            g = dist.new_group([pred, succ])
            if rank == pred:
                st.pred_group = g
            if rank == succ:
                st.succ_group = g
    _STATE = st
    return topo


def model_parallel_is_initialized() -> bool:
    return _STATE is not None


def destroy_model_parallel() -> None:
    global _STATE
    _STATE = None


def _st() -> _State:
    """Current state; a process that never initialised torch.distributed is treated as
    the single rank of a 1x1x1 layout so that layers can be built in plain scripts."""
    global _STATE
    if _STATE is None:
        if dist.is_available() and dist.is_initialized():
            raise AssertionError("call initialize_model_parallel first")
        return _State(Topology(1, 1, 1), 0)
    return _STATE


def get_topology() -> Topology:
    return _st().topo


def get_model_parallel_group():
    return _st().tp_group


def get_data_parallel_group():
    return _st().dp_group


def get_pipeline_parallel_group():
    return _st().pp_group


def get_model_parallel_world_size() -> int:
    return _st().topo.tp


def get_model_parallel_rank() -> int:
    return _st().tp_idx


def get_model_parallel_src_rank() -> int:
    s = _st()
    return s.topo.tp_src_rank(s.rank)


def get_model_parallel_dst_rank() -> int:
    s = _st()
    return s.topo.tp_dst_rank(s.rank)


def get_model_parallel_next_src_rank() -> Optional[int]:
    s = _st()
    return s.topo.tp_src_rank(s.rank) + s.topo.tp if s.pp_idx < s.topo.pp - 1 else None


def get_model_parallel_prev_dst_rank() -> Optional[int]:
    s = _st()
    return s.topo.tp_dst_rank(s.rank) - s.topo.tp if s.pp_idx > 0 else None


def get_data_parallel_world_size() -> int:
    return _st().topo.dp


def get_data_parallel_rank() -> int:
    return _st().dp_idx


def get_pipeline_parallel_world_size() -> int:
    return _st().topo.pp


def get_pipeline_parallel_group_rank() -> int:
    return _st().pp_idx


def get_pipeline_parallel_pred_group():
    return _st().pred_group


def get_pipeline_parallel_succ_group():
    return _st().succ_group


def get_pipeline_prev_rank() -> Optional[int]:
    s = _st()
    return s.topo.prev_stage_rank(s.rank)


def get_pipeline_next_rank() -> Optional[int]:
    s = _st()
    return s.topo.next_stage_rank(s.rank)
