"""Analytic latency model of one layer and one token slice on a B200, built from the measured
behaviour of this package's kernels.

Why it exists.  The planner (``latency_model.py``) needs a table ``(batch, slice, context) ->
forward / backward / update time`` of ONE layer.  The reference measures that table by running
a layer eagerly (terapipe_latency_model.py:17-225); on a B200 an eagerly launched layer of a
short slice is bound by launch overhead, not by the kernels, so a table measured that way makes
every slice look equally cheap and the dynamic program drifts to schedules that lose against
uniform slices.  Inside a training step the kernels run back to back (CUDA graph or a full
queue), and their times follow from a handful of measured constants:

* GEMMs: cycles = set-up + waves x main loop of one tile (proportional to K) + exposed epilogue
  of the last tile, for the tile shapes of ``csrc/gemm_sm100.cu`` (the same table as its
  ``pick_tile``), at the SM clock seen under load;
* attention: a fixed part plus a cost per 128-key (forward, dQ) or 128-query (dK/dV) block and
  wave of CTAs;
* LayerNorm and the all-reduce: a fixed part plus bytes over an effective bandwidth.

``synthesize_latency_table`` writes a table in the measurer's JSON schema, so the fit, the
dynamic program and ``dp_results.json`` are produced by exactly the same code as for a measured
table.  ``predict_iteration_ms`` applies the model to a whole schedule (pipeline fill + steady
state + deferred weight gradients + optimizer) and is what the calibration is checked against.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from ..models.config import MODEL_CONFIGS


@dataclass
class B200KernelModel:
    # ---- clocks and launches
    sm_mhz: float = 1792.0          # median SM clock during a step (power capped)
    launch_us: float = 5.0          # kernel-to-kernel gap + prologue not covered by the cycle counts
    n_sms: int = 148
    # ---- GEMM (kilo-cycles; same candidates as pick_tile in csrc/gemm_sm100.cu)
    gemm_setup_kc: float = 2.7
    gemm_cold_l2: float = 1.2       # operands of a step are cold in L2: main loop slow-down
    gemm_long_k: float = 1.45       # K >= 8192: DRAM streaming and power cap stretch the main loop
    # ---- attention (micro-seconds per block of 128 keys / queries and wave of CTAs)
    attn_fixed_us: float = 1.6
    attn_fwd_block_us: float = 1.9
    attn_dq_block_us: float = 2.7
    attn_dkdv_block_us: float = 3.5
    attn_bwd_fixed_us: float = 2.5
    attn_delta_us: float = 6.6
    # ---- memory-bound kernels (effective TB/s for a 1024-row slice) and collectives
    ln_fwd_tbs: float = 1.6
    ln_bwd_tbs: float = 0.9
    colsum_tbs: float = 4.0
    adam_gbs: float = 5716.0
    allreduce_base_us: float = 25.0   # NCCL all-reduce of an activation tile inside a TP group
    allreduce_gbs: float = 280.0
    fused_allreduce_extra_us: float = 50.0  # fused GEMM + all-reduce: tail after the last MMA
    p2p_base_us: float = 12.0
    p2p_gbs: float = 400.0

    # (tile rows, tile cols, CTA pair?, main loop kc per 2048 of K, epilogue per tile kc, tail kc)
    _TILES = ((256, 256, True, 16.7, 0.0, 8.5), (256, 128, True, 10.0, 0.0, 5.5),
              (256, 256, False, 36.0, 18.0, 0.0), (128, 256, False, 24.7, 0.0, 10.0),
              (128, 128, False, 16.4, 0.0, 5.4), (128, 64, False, 9.5, 0.0, 3.0))

    def _us(self, kilo_cycles: float) -> float:
        return kilo_cycles * 1e3 / self.sm_mhz

    # ------------------------------------------------------------------ kernels
    def gemm_us(self, M: int, N: int, K: int) -> float:
        """``[M, K] x [N, K]^T`` with the tile that minimises the modelled time."""
        if min(M, N, K) <= 0:
            return 0.0
        stretch = self.gemm_long_k if K >= 8192 else self.gemm_cold_l2
        best = math.inf
        for bm, bn, pair, loop, epi_each, tail in self._TILES:
            tiles = math.ceil(M / bm) * math.ceil(N / bn)
            slots = self.n_sms // 2 if pair else self.n_sms
            waves = math.ceil(tiles / slots)
            best = min(best, waves * (loop * stretch * K / 2048.0 + epi_each) + tail)
        return self.launch_us + self._us(self.gemm_setup_kc + best)

    def _attn_waves(self, b: int, heads: int, q_rows: int) -> int:
        return math.ceil(b * heads * math.ceil(q_rows / 128) / self.n_sms)

    def attn_fwd_us(self, b: int, heads: int, t: int, c: int) -> float:
        blocks = math.ceil((c + t) / 128)
        return self.launch_us + self._attn_waves(b, heads, t) * (self.attn_fixed_us + self.attn_fwd_block_us * blocks)

    def attn_bwd_us(self, b: int, heads: int, t: int, c: int, seq_len: int) -> float:
        """delta + dK/dV of the slice's keys over all later queries + dQ over all earlier keys."""
        dq = self._attn_waves(b, heads, t) * (self.attn_bwd_fixed_us + self.attn_dq_block_us * math.ceil((c + t) / 128))
        dkdv = self._attn_waves(b, heads, t) * (self.attn_bwd_fixed_us +
                                                self.attn_dkdv_block_us * math.ceil((seq_len - c) / 128))
        return 2 * self.launch_us + self.attn_delta_us + dq + dkdv

    def layernorm_us(self, rows: int, H: int, backward: bool) -> float:
        bytes_ = rows * H * 2 * (4 if backward else 2)
        return self.launch_us + bytes_ / ((self.ln_bwd_tbs if backward else self.ln_fwd_tbs) * 1e6)

    def allreduce_us(self, rows: int, H: int, tp: int, fused: bool) -> float:
        if tp <= 1:
            return 0.0
        if fused:
            return self.fused_allreduce_extra_us
        wire = 2.0 * (tp - 1) / tp * rows * H * 2
        return self.allreduce_base_us + wire / (self.allreduce_gbs * 1e3)

    def p2p_us(self, rows: int, H: int) -> float:
        return self.p2p_base_us + rows * H * 2 / (self.p2p_gbs * 1e3)

    # ------------------------------------------------------------------ one layer, one slice
    def layer_slice_us(self, H: int, heads: int, seq_len: int, tp: int, b: int, t: int, c: int,
                       fused_tp: bool = False) -> Tuple[float, float]:
        """(forward, backward) time of one layer for a slice of ``t`` tokens x ``b`` sequences
        attending over ``c`` cached tokens; weight gradients are not included (they run once per
        layer over the whole sequence, see ``layer_update_us``)."""
        rows, h_loc, F_ = b * t, heads // tp, 4 * H
        ar = self.allreduce_us(rows, H, tp, fused_tp)
        fwd = (self.layernorm_us(rows, H, False) + self.gemm_us(rows, 3 * H // tp, H) +
               self.attn_fwd_us(b, h_loc, t, c) + self.gemm_us(rows, H, H // tp) + ar +
               self.layernorm_us(rows, H, False) + self.gemm_us(rows, F_ // tp, H) +
               self.gemm_us(rows, H, F_ // tp) + ar)
        bwd = (self.gemm_us(rows, F_ // tp, H) + self.gemm_us(rows, H, F_ // tp) + ar +
               self.layernorm_us(rows, H, True) + self.gemm_us(rows, H // tp, H) +
               self.attn_bwd_us(b, h_loc, t, c, seq_len) + self.gemm_us(rows, H, 3 * H // tp) + ar +
               self.layernorm_us(rows, H, True))
        return fwd, bwd

    def layer_update_us(self, H: int, tp: int, total_rows: int) -> float:
        """Per layer and iteration: the four whole-sequence weight-gradient GEMMs, the bias
        column sums and this layer's share of the fused Adam."""
        F_ = 4 * H
        wgrad = (self.gemm_us(3 * H // tp, H, total_rows) + self.gemm_us(H, H // tp, total_rows) +
                 self.gemm_us(F_ // tp, H, total_rows) + self.gemm_us(H, F_ // tp, total_rows))
        colsum = sum(self.launch_us + total_rows * n * 2 / (self.colsum_tbs * 1e6)
                     for n in (3 * H // tp, H, F_ // tp, H))
        params = 12 * H * H / tp
        return wgrad + colsum + params * 34 / (self.adam_gbs * 1e3)


def predict_iteration_ms(model_name: str, batch: int, tp: int, pp: int, batch_slices: Sequence[int],
                         seq_slices: Sequence[int], km: Optional[B200KernelModel] = None,
                         fused_tp: bool = False, n_layers: Optional[int] = None) -> float:
    """Iteration time of the token-slice pipeline under the kernel model: every slice passes the
    ``pp`` stages forward, then backward in reverse order; the pipeline adds ``pp - 1`` times the
    longest slice to each pass; the first stage then runs its deferred weight gradients."""
    km = km or B200KernelModel()
    layers, H, seq_len, heads = MODEL_CONFIGS[model_name]
    layers = n_layers if n_layers is not None else layers
    per_stage = math.ceil(layers / pp)
    f_total = b_total = f_max = b_max = 0.0
    for b in batch_slices:
        c = 0
        for t in seq_slices:
            f, bw = km.layer_slice_us(H, heads, seq_len, tp, b, t, c, fused_tp)
            comm = km.p2p_us(b * t, H) if pp > 1 else 0.0
            f, bw = f * per_stage + comm, bw * per_stage + comm
            f_total, b_total = f_total + f, b_total + bw
            f_max, b_max = max(f_max, f), max(b_max, bw)
            c += t
    update = km.layer_update_us(H, tp, batch * seq_len) * per_stage
    return (f_total + b_total + (pp - 1) * (f_max + b_max) + update) / 1e3


def synthesize_latency_table(model_name: str, tp: int, batch_sizes: Iterable[int], step: int = 64,
                             km: Optional[B200KernelModel] = None, fused_tp: bool = False,
                             total_batch: Optional[int] = None) -> Dict[str, dict]:
    """A latency table in the schema of the measurer (keys ``"b_s_c"``, times in seconds) for
    every batch size, slice length and context length on a grid of ``step`` tokens."""
    km = km or B200KernelModel()
    _, H, seq_len, heads = MODEL_CONFIGS[model_name]
    batch_sizes = list(batch_sizes)
    rows_total = (total_batch or max(batch_sizes)) * seq_len
    update = km.layer_update_us(H, tp, rows_total)
    table: Dict[str, dict] = {}
    for b in batch_sizes:
        for s in range(step, seq_len + 1, step):
            for c in range(0, seq_len - s + 1, step):
                f, bw = km.layer_slice_us(H, heads, seq_len, tp, b, s, c, fused_tp)
                table[f"{b}_{s}_{c}"] = {
                    "py_forward_mean": 0.0, "py_forward_std": 0.0, "forward_mean": f * 1e-6,
                    "forward_std": 0.0, "py_backward_mean": 0.0, "py_backward_std": 0.0,
                    "backward_mean": bw * 1e-6, "backward_std": 0.0,
                    "update_mean": update * 1e-6, "update_std": 0.0}
    return table


def write_tables(model_name: str, tp: int, batch_sizes: Iterable[int], data_dir: str, step: int = 64,
                 km: Optional[B200KernelModel] = None, fused_tp: bool = False,
                 total_batch: Optional[int] = None) -> List[str]:
    """Write ``latency_model.<model>.mp_<tp>.json`` and ``<model>.communication_latency.json``
    (inter-stage transfer times, in tokens) into ``data_dir``; returns the two paths."""
    km = km or B200KernelModel()
    os.makedirs(data_dir, exist_ok=True)
    _, H, seq_len, _ = MODEL_CONFIGS[model_name]
    table = synthesize_latency_table(model_name, tp, batch_sizes, step, km, fused_tp, total_batch)
    p1 = os.path.join(data_dir, f"latency_model.{model_name}.mp_{tp}.json")
    with open(p1, "w") as f:
        json.dump(table, f)
    sizes = [1 << i for i in range(0, int(math.log2(seq_len * max(batch_sizes))) + 1)]
    comm = {"tensor_sizes": sizes, "mean": [km.p2p_us(n, H) * 1e-6 for n in sizes],
            "std": [0.0 for _ in sizes]}
    p2 = os.path.join(data_dir, f"{model_name}.communication_latency.json")
    with open(p2, "w") as f:
        json.dump(comm, f)
    return [p1, p2]
