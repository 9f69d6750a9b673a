"""Analytic FLOP count of one training iteration and efficiency against a device peak.

``flop_stats`` counts multiply-adds of LayerNorm, QKV, scaling, QK^T, softmax, PV,
output projection and the FFN, times 6 (2 FLOP per multiply-add, forward + 2x backward),
as the reference does (flop_model.py:4-42), so its numbers are comparable.
"""
from __future__ import annotations

from ..models.config import MODEL_CONFIGS

V100_FP16_TFLOPS = 112.0
B200_BF16_TFLOPS_MEASURED = 1638.7   # cuBLAS bf16 8192^3 burst on this pool's B200s


def layer_muladds(batch_size: int, seq_len: int, hidden: int, heads: int) -> float:
    c = batch_size * seq_len * hidden
    a = batch_size * heads * seq_len * seq_len
    attention = (c + 3 * c * hidden + c) + (a * (hidden / heads) + a) + (c * hidden + c)
    ffn = 4 * c * hidden + 4 * c + 4 * c * hidden
    return attention + ffn


def flop_stats(model_name: str, batch_size: int, n_layers=None) -> float:
    """GFLOP of one iteration (forward + backward) over the whole model."""
    layers, hidden, seq_len, heads = MODEL_CONFIGS[model_name]
    layers = n_layers if n_layers is not None else layers
    return 6 * layer_muladds(batch_size, seq_len, hidden, heads) * layers / 1e9


def slice_flops(batch: int, t: int, c: int, hidden: int, heads_local: int, head_dim: int,
                tp: int = 1) -> float:
    """Forward FLOP of one layer on one token slice: GEMMs plus causal attention over
    ``c`` cached and ``t`` own positions."""
    tokens = batch * t
    gemm = 24.0 * tokens * hidden * hidden / tp
    attn = 4.0 * batch * heads_local * t * (c + t) * head_dim
    return gemm + attn


def efficiency(model_name, batch_size, n_gpus, latency, peak_tflops=B200_BF16_TFLOPS_MEASURED,
               n_layers=None) -> float:
    """Fraction of ``peak_tflops * n_gpus`` sustained by an iteration of ``latency`` s."""
    return flop_stats(model_name, batch_size, n_layers) / 1000.0 / (peak_tflops * n_gpus * latency)


def efficiency_stats(model_name, batch_size, n_gpus, latency, n_slices, n_stages, method_name,
                     peak_tflops=V100_FP16_TFLOPS, printer=print):
    eff = efficiency(model_name, batch_size, n_gpus, latency, peak_tflops)
    printer(f"[{method_name}] {model_name} efficiency={eff:.4f} "
            f"({eff * peak_tflops:.4f} TFlops of {peak_tflops:g} TFlops) "
            f"theoretical-pipeline-efficiency = {n_slices / (n_stages + n_slices - 1):.4f}")
    return eff


# iteration latencies published with the reference (V100 clusters), flop_model.py:62-68
PUBLISHED = [
    ("gpt3-175b", 2, 384, 1.160, 32, 48, "w/ TeraPipe"),
    ("gpt3-175b", 2, 384, 5.822, 2, 48, "w/o TeraPipe"),
    ("gpt3-13b", 32, 320, 1.328, 96, 40, "w/ TeraPipe"),
    ("gpt3-13b", 32, 320, 1.863, 32, 40, "w/o TeraPipe"),
    ("gpt3-1b", 128, 192, 0.913, 72, 24, "Both"),
]


def main():
    for row in PUBLISHED:
        efficiency_stats(*row)


if __name__ == "__main__":
    main()
