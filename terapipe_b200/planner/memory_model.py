"""Analytic peak-memory models.

``peak_memory_per_gpu`` is the reference's unfused model (memory_model.py:4-82): fp16
activations incl. materialised ``[B*heads, L, L]`` fp16 scores and fp32 probabilities,
and 14 bytes of parameter state per parameter.  ``engine_memory_per_gpu`` models the
sm_100a engine instead: no score/probability storage (fused attention), fp32 main grads
(18 bytes per parameter), full-length 16-bit gradient buffers per layer, and it takes plain
GPU counts, so it is defined for 1, 2 or 4 GPUs as well.
"""
from __future__ import annotations

from ..models.config import MODEL_CONFIGS

_F16, _F32 = 2, 4


def _layer_params(hidden: int, m: float) -> float:
    attn = 2 * hidden + (hidden * hidden + hidden) * 3 / m + (hidden * hidden + hidden) / m
    ffn = 2 * hidden + (hidden * hidden + hidden) * 4 / m + (hidden * 4 * hidden + hidden) / m
    return attn + ffn


def peak_memory_per_gpu(model_name, batch_size, n_nodes, n_data_parallel_replicas=1,
                        gpus_per_megatronlm_shard=8, gpus_per_node=8, verbose=False) -> float:
    """Peak GB per GPU of the unfused runtime; ``inf`` when the layout does not divide."""
    n_layers, hidden, seq_len, heads = MODEL_CONFIGS[model_name]
    m = gpus_per_megatronlm_shard
    if (n_nodes <= 0 or n_layers % n_nodes or gpus_per_node % m
            or (n_nodes * gpus_per_node) % n_data_parallel_replicas):
        if verbose:
            print("layout does not divide", flush=True)
        return float("inf")
    layers_per_shard = n_layers / (n_nodes * gpus_per_node) * (m * n_data_parallel_replicas)
    c = batch_size * seq_len * hidden * _F16
    a = batch_size * heads * seq_len * seq_len
    attn_act = (c + 3 * c / m + c / m) + a / m * (_F16 + _F32) + (c / m + c)
    ffn_act = c + 4 * c / m + c
    n_params = _layer_params(hidden, m)
    param_bytes = n_params * (_F16 + _F32 + 2 * _F32)
    layer_bytes = param_bytes + max(attn_act + ffn_act, n_params * _F32)
    return (2 * c + layer_bytes * layers_per_shard) / 2 ** 30


def memory_stats(model_name, batch_size, printer=print):
    n_layers, hidden, seq_len, heads = MODEL_CONFIGS[model_name]
    c = batch_size * seq_len * hidden * _F16
    a = batch_size * heads * seq_len * seq_len
    act = (c + 3 * c + c) + a * (_F16 + _F32) + (c + c) + (c + 4 * c + c)
    params = _layer_params(hidden, 1) * (_F16 + 3 * _F32)
    printer(f"{model_name}: activation size = {n_layers * act / 2 ** 30} GB, "
            f"parameter size = {params * n_layers / 2 ** 30} GB")
    return n_layers * act / 2 ** 30, params * n_layers / 2 ** 30


def engine_memory_per_gpu(model_name, batch_size, tp=1, pp=1, n_layers=None,
                          keep_gelu_input=True) -> float:
    """Peak GB per GPU of the sm_100a engine for one data-parallel replica.

    Per layer and token the engine keeps (16-bit unless noted): the layer input, both LayerNorm
    outputs and the post-attention residual stream (4H, replicated over TP); 1/tp of QKV (3H),
    of the attention output (H) and of the FFN activation (4H, twice when GeLU keeps its input);
    the full-length gradient buffers of the layer output and of the post-attention stream (2H)
    and 1/tp of those of the FFN pre-activation (4H), QKV (3H) and attention output (H);
    LayerNorm statistics (4 fp32) and log-sum-exp / delta rows (2 fp32 per local head).
    Parameters cost 18 bytes each (16-bit model, fp32 master, two Adam moments, fp32 gradient).
    Heads that are not 64 or 128 wide are stored 128 wide: QKV, the attention output, their
    gradients and the two attention projection matrices grow by 128 / head_dim."""
    layers, hidden, seq_len, heads = MODEL_CONFIGS[model_name]
    layers = n_layers if n_layers is not None else layers
    per_stage = -(-layers // pp)
    tokens = batch_size * seq_len
    head_dim = hidden // heads
    pad = 1.0 if head_dim in (64, 128) else (64 if head_dim < 64 else 128) / head_dim
    attn_w = (3 * hidden + hidden) * pad
    act_elems = 4 * hidden + (attn_w + (8 if keep_gelu_input else 4) * hidden) / tp
    grad_elems = 2 * hidden + (4 * hidden + attn_w) / tp
    act = tokens * (act_elems + grad_elems) * _F16 + tokens * (4 + 2 * heads / tp) * _F32
    params = (_layer_params(hidden, tp) + (pad - 1.0) * 4 * hidden * hidden / tp) * (_F16 + 4 * _F32)
    io = 4 * tokens * hidden * _F16
    return (per_stage * (act + params) + io) / 2 ** 30


if __name__ == "__main__":
    print(peak_memory_per_gpu("gpt3-175b", 1, 32))
    print(peak_memory_per_gpu("gpt3-175b", 1, 48))
    memory_stats("gpt3-175b", 1536)
    memory_stats("gpt3-175b", 2)
