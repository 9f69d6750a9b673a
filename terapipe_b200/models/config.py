"""Model registry and the per-run transformer configuration.

The registry keeps the names and (n_layers, hidden, seq_len, n_heads) tuples of the
reference (transformer_models.py:17-59) and its latency-table batch sizes
(transformer_models.py:61-69) so that run scripts and planner inputs written for the
reference keep working.  The FFN width is always 4 * hidden.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Tuple

import torch

NEG_INF = -65504  # most negative finite fp16 value; additive causal mask fill


def _registry() -> Dict[str, Tuple[int, int, int, int]]:
    # name: layers hidden seq head_dim   (heads = hidden // head_dim)
    table = """
    test 24 256 128 64
    test-l512 512 256 128 64
    test-s1024 48 2048 1024 64
    test-s2048 48 2048 2048 64
    test-h3072 48 3072 2048 64
    gpt2-1hm 12 768 1024 64
    gpt2-3hm 24 1024 1024 64
    gpt2-7hm 36 1280 1024 64
    gpt2-1b 48 1600 1024 64
    megatron-1b 40 1536 1024 96
    megatron-2b 54 1920 1024 96
    megatron-4b 64 2304 1024 96
    megatron-8b 72 3072 1024 96
    gpt3-1hm 12 768 2048 64
    gpt3-3hm 24 1024 2048 64
    gpt3-7hm 24 1536 2048 96
    gpt3-1b 24 2048 2048 128
    gpt3-2b 32 2560 2048 80
    gpt3-6b 32 4096 2048 128
    gpt3-13b 40 5120 2048 128
    gpt3-44b 96 6144 2048 128
    gpt3-175b 96 12288 2048 128
    gpt3-13b-4096 40 5120 4096 128
    gpt3-13b-6144 40 5120 6144 128
    gpt3-13b-8192 40 5120 8192 128
    gpt2-1hm-single-device 10 768 2048 64
    gpt2-3hm-single-device 8 1024 2048 64
    gpt2-7hm-single-device 6 1280 2048 64
    gpt2-1b-single-device 4 1600 2048 64
    gpt3-1b-single-device 5 2048 2048 128
    gpt3-2b-single-device 3 2560 2048 80
    gpt3-6b-single-device 2 4096 2048 128
    gpt3-13b-single-device 1 5120 2048 128
    gpt3-175b-single-node 2 12288 2048 128
    """
    out = {}
    for line in table.strip().splitlines():
        name, n_layers, hidden, seq, head_dim = line.split()
        out[name] = (int(n_layers), int(hidden), int(seq), int(hidden) // int(head_dim))
    # the one entry whose head count is given directly (half-width 175B with 384 heads)
    out["gpt3-175b-megatron"] = (48, 12288 // 2, 2048, 384)
    return out


MODEL_CONFIGS: Dict[str, Tuple[int, int, int, int]] = _registry()

# largest batch measured per model when building latency tables
BATCH_CONFIGS: Dict[str, int] = {
    "gpt3-1b": 72, "gpt3-13b": 32, "gpt3-44b": 16, "gpt3-175b": 2,
    "gpt3-13b-4096": 8, "gpt3-13b-6144": 4, "gpt3-13b-8192": 2,
}


@dataclasses.dataclass
class TransformerConfig:
    """Shape of one benchmark run (reference: transformer_models.py:71-174).

    Activations are sequence-first ``[seq, batch, hidden]``.  ``activation`` selects
    the FFN nonlinearity: ``"gelu"`` (default) or ``"relu"`` (what the reference
    layer computes, transformer_models.py:282).
    """
    batch_size: int = 1
    seq_len: int = 1024
    n_layers: int = 12
    embedding_dim: int = 768
    ffn_embedding_dim: Optional[int] = None
    num_attention_heads: Optional[int] = None
    placement_orders: Optional[list] = None
    n_devices: Optional[int] = None
    model_name: Optional[str] = None
    activation: str = "gelu"

    def __post_init__(self):
        if self.model_name is not None:
            (self.n_layers, self.embedding_dim, self.seq_len,
             self.num_attention_heads) = MODEL_CONFIGS[self.model_name]
            self.ffn_embedding_dim = 4 * self.embedding_dim
        if not self.ffn_embedding_dim:
            self.ffn_embedding_dim = 4 * self.embedding_dim
        if not self.num_attention_heads:
            self.num_attention_heads = self.embedding_dim // 64
        if self.n_devices is None:
            self.n_devices = torch.cuda.device_count() if torch.cuda.is_available() else 1
        if self.placement_orders is None:
            self.placement_orders = list(range(self.n_devices))
        if self.activation not in ("gelu", "relu"):
            raise ValueError(f"unknown activation {self.activation!r}")

    @classmethod
    def from_predefined_model(cls, model_name, n_devices=None, batch_size=1,
                              n_layers=None, activation="gelu"):
        cfg = cls(batch_size=batch_size, n_devices=n_devices, model_name=model_name,
                  activation=activation)
        cfg.model_name = model_name
        if n_layers is not None:  # truncated stacks (e.g. 8 layers of 175B width)
            cfg.n_layers = int(n_layers)
        return cfg

    @property
    def attention_heads_dim(self) -> int:
        return self.embedding_dim // self.num_attention_heads

    # ---- input factories -------------------------------------------------------
    def _device(self, device):
        if device is None:
            return "cuda" if torch.cuda.is_available() else "cpu"
        return device

    def create_inputs(self, device=None, requires_grad=False, dtype=torch.float32,
                      generator=None):
        x = torch.randn(self.seq_len, self.batch_size, self.embedding_dim,
                        device=self._device(device), dtype=dtype, generator=generator)
        return x.requires_grad_(requires_grad)

    def create_inputs_empty(self, device=None, dtype=torch.float32):
        return torch.empty(self.seq_len, self.batch_size, self.embedding_dim,
                           device=self._device(device), dtype=dtype)

    def create_pseudo_inputs_outputs(self, device=None, inputs_requires_grad=False):
        dev = self._device(device)
        x = torch.randn(self.seq_len, self.batch_size, self.embedding_dim, device=dev)
        tail = torch.randn(1, self.batch_size, self.embedding_dim, device=dev)
        return x.requires_grad_(inputs_requires_grad), torch.cat([x[1:].detach(), tail])

    def create_pseudo_attention_cache(self, length, device=None, requires_grad=False):
        dev = self._device(device)
        shape = (self.batch_size * self.num_attention_heads, length, self.attention_heads_dim)
        return [{name: torch.randn(shape, device=dev).requires_grad_(requires_grad)
                 for name in ("k", "v")} for _ in range(self.n_layers)]

    @staticmethod
    def compute_pseudo_loss(pred_y, y):
        return torch.mean((pred_y - y) ** 2)

    # ---- legacy layer factories (single process; transformer_models.py:113-174) --------
    def _make_layer(self, device):
        from .layers import TransformerLayer
        return TransformerLayer(self.embedding_dim, self.ffn_embedding_dim,
                                self.num_attention_heads, device=device,
                                activation=self.activation)

    def create_layers_and_inputs(self):
        layers = [self._make_layer("cpu") for _ in range(self.n_layers)]
        return layers, torch.randn(self.seq_len, self.batch_size, self.embedding_dim)

    def create_layers_gpu(self, device=None):
        dev = self._device(device)
        return [self._make_layer(dev) for _ in range(self.n_layers // self.n_devices)]

    def create_layers_and_inputs_on_gpu(self):
        if self.n_layers % self.n_devices:
            raise AssertionError("layers must divide evenly over the devices")
        per_dev = self.n_layers // self.n_devices
        cuda = torch.cuda.is_available()
        devs = [f"cuda:{self.placement_orders[i // per_dev]}" if cuda else "cpu"
                for i in range(self.n_layers)]
        layers = [self._make_layer(d) for d in devs]
        x = torch.randn(self.seq_len, self.batch_size, self.embedding_dim, device=devs[0])
        return layers, x

    def n_params_per_layer(self) -> int:
        h, f = self.embedding_dim, self.ffn_embedding_dim
        return 4 * h + (3 * h * h + 3 * h) + (h * h + h) + (f * h + f) + (h * f + h)
