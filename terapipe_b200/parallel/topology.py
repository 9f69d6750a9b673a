"""Pure-arithmetic rank layout: tensor-parallel fastest, then pipeline, then data.

Global rank = dp_idx * (tp * pp) + pp_idx * tp + tp_idx, the layout of the reference
(mpu/initialize.py:42-105).  Nothing here touches torch.distributed, so the layout
can be unit-tested for any world size on a machine without GPUs.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class Topology:
    world_size: int
    tp: int
    pp: int

    def __post_init__(self):
        if self.tp < 1 or self.pp < 1:
            raise ValueError("parallel sizes must be positive")
        if self.world_size % (self.tp * self.pp):
            raise ValueError(
                f"world size {self.world_size} is not divisible by tp*pp = {self.tp * self.pp}")

    @property
    def dp(self) -> int:
        return self.world_size // (self.tp * self.pp)

    @property
    def block(self) -> int:
        """Ranks per data-parallel replica."""
        return self.tp * self.pp

    # ---- coordinates ----------------------------------------------------------
    def coords(self, rank: int) -> Tuple[int, int, int]:
        """(dp_idx, pp_idx, tp_idx) of a global rank."""
        return rank // self.block, (rank // self.tp) % self.pp, rank % self.tp

    def rank_of(self, dp_idx: int, pp_idx: int, tp_idx: int) -> int:
        return dp_idx * self.block + pp_idx * self.tp + tp_idx

    # ---- groups ---------------------------------------------------------------
    def dp_groups(self) -> List[List[int]]:
        return [list(range(i, self.world_size, self.block)) for i in range(self.block)]

    def tp_groups(self) -> List[List[int]]:
        return [list(range(i * self.tp, (i + 1) * self.tp))
                for i in range(self.world_size // self.tp)]

    def pp_groups(self) -> List[List[int]]:
        """One group per (dp_idx, tp_idx): the ranks holding the same shard of every stage."""
        return [[self.rank_of(d, s, t) for s in range(self.pp)]
                for d in range(self.dp) for t in range(self.tp)]

    def stage_pairs(self) -> List[Tuple[int, int]]:
        """(pred, succ) rank pairs joined by a shard-to-shard pipeline link."""
        return [(self.rank_of(d, s - 1, t), self.rank_of(d, s, t))
                for d in range(self.dp) for s in range(1, self.pp) for t in range(self.tp)]

    def reference_stage_pairs(self) -> List[Tuple[int, int]]:
        """The reference's links: last TP rank of a stage to first TP rank of the next."""
        return [(d * self.block + s * self.tp - 1, d * self.block + s * self.tp)
                for d in range(self.dp) for s in range(1, self.pp)]

    # ---- neighbours -----------------------------------------------------------
    def tp_src_rank(self, rank: int) -> int:
        return (rank // self.tp) * self.tp

    def tp_dst_rank(self, rank: int) -> int:
        return self.tp_src_rank(rank) + self.tp - 1

    def prev_stage_rank(self, rank: int) -> Optional[int]:
        return rank - self.tp if self.coords(rank)[1] > 0 else None

    def next_stage_rank(self, rank: int) -> Optional[int]:
        return rank + self.tp if self.coords(rank)[1] < self.pp - 1 else None

    # ---- layers ---------------------------------------------------------------
    def layers_of_stage(self, n_layers: int, pp_idx: int) -> range:
        """Global layer ids of a stage; the first ``n_layers % pp`` stages hold one more
        (terapipe.py:276-279, :320-323)."""
        base, rem = divmod(n_layers, self.pp)
        start = pp_idx * base + min(pp_idx, rem)
        return range(start, start + base + (1 if pp_idx < rem else 0))
