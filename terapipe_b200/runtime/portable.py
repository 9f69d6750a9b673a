"""Portable token-slice pipeline on torch autograd (CPU/gloo or any CUDA device).

Schedule of the reference's production runtime (test_transformer_terapipe.py:107-175,
:270-287): for every batch slice all token slices go forward in order; backward walks
batch slices and token slices in reverse; then the data-parallel all-reduce and the
optimizer.  Differences in mechanism, not in result:

* The KV cache is a plain buffer; slice *j* differentiates w.r.t. a detached view of the
  prefix rows and its own new rows, and prefix gradients are added into a persistent
  fp32 ``dK/dV`` accumulator (instead of cloning a full-length gradient cache per layer
  per slice, transformer_models.py:186-190).
* Parameter gradients accumulate in fp32 main-grad tensors.
* The seed gradient of ``loss = mean(output)`` is the constant ``scale / numel``.

This path is the oracle for the sm_100a engine and the multi-process test bed.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist
from torch import nn

from .. import parallel as mpu
from ..models import TransformerConfig, TransformerLayer, grid_slice_batch_and_sequence
from ..parallel import p2p
from ..utils import set_random_seed

LOSS_SCALE_FACTOR = 128.0


class TransformerLayers(nn.Module):
    """The layers of one pipeline stage; state-dict keys ``layers.<local id>.<param>``."""

    def __init__(self, n_layers, embedding_dim, ffn_embedding_dim, num_attention_heads,
                 mixed_precision=False, device="cpu", checkpoint_gradients=False,
                 activation="gelu", dtype=torch.float16, sequence_parallel=False):
        super().__init__()
        self.layers = nn.ModuleList([
            TransformerLayer(embedding_dim, ffn_embedding_dim, num_attention_heads, device=device,
                             checkpoint_gradients=checkpoint_gradients, activation=activation,
                             sequence_parallel=sequence_parallel)
            for _ in range(n_layers)])
        if mixed_precision:
            self.to(dtype)

    def create_cache(self, batch_size, seq_len):
        p = next(self.parameters())
        return [layer.attn.create_attn_cache(batch_size, seq_len, p.device, p.dtype)
                for layer in self.layers]

    def forward(self, x, cache, cache_len):
        new_cache = []
        for layer, kv in zip(self.layers, cache):
            x, kv_out = layer(x, kv, cache_len)
            new_cache.append(kv_out)
        return x, new_cache


class PortablePipeline:
    """One rank of a TP x PP x DP job on the portable path."""

    def __init__(self, config: TransformerConfig, batch_slices: Sequence[int],
                 seq_slices: Sequence[int], mixed_precision=False, checkpoint_gradients=False,
                 device: Optional[str] = None, dtype=torch.float16, seed: int = 0, lr=1e-10,
                 loss_scale: float = LOSS_SCALE_FACTOR, sequence_parallel: bool = False):
        """``sequence_parallel``: between the GEMM pairs every tensor-parallel rank keeps only
        its chunk of a slice's tokens (LayerNorm, residual stream, and what travels between
        pipeline stages: 1/tp of the bytes per link); slice lengths must divide by tp."""
        self.config = config
        self.batch_slices, self.seq_slices = list(batch_slices), list(seq_slices)
        self.mixed_precision = mixed_precision
        self.low_dtype = dtype if mixed_precision else torch.float32
        self.loss_scale = loss_scale if mixed_precision else 1.0
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.topo = mpu.get_topology()
        self.sequence_parallel = bool(sequence_parallel) and self.topo.tp > 1
        if self.sequence_parallel and any(t % self.topo.tp for t in self.seq_slices):
            raise ValueError("sequence_parallel needs slice lengths divisible by the tensor-parallel size")
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.dp_idx, self.pp_idx, self.tp_idx = self.topo.coords(self.rank)
        self.is_first, self.is_last = self.pp_idx == 0, self.pp_idx == self.topo.pp - 1
        self.layer_ids = self.topo.layers_of_stage(config.n_layers, self.pp_idx)
        self.seed = seed

        set_random_seed(seed)
        # every stage draws the weights of all earlier layers first so that a layer's
        # values do not depend on how the stack is cut into stages
        self._skip_rng_for_layers(self.layer_ids.start)
        self.layers = TransformerLayers(
            len(self.layer_ids), config.embedding_dim, config.ffn_embedding_dim,
            config.num_attention_heads, mixed_precision, self.device, checkpoint_gradients,
            config.activation, dtype, sequence_parallel=self.sequence_parallel)
        self.params: List[torch.Tensor] = list(self.layers.parameters())
        # parameters replicated over the TP group whose gradients are partial (per token chunk)
        # under sequence parallelism: LayerNorm weights / biases, biases of row-parallel layers
        self._partial_grad_ids = [i for i, (n, _) in enumerate(self.layers.named_parameters())
                                  if n.endswith(("attn_ln.weight", "attn_ln.bias", "fc_ln.weight",
                                                 "fc_ln.bias", "out_proj.bias", "fc2.bias"))] \
            if self.sequence_parallel else []
        self.main_grads = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        if mixed_precision:
            self.master = [p.detach().clone().float().requires_grad_() for p in self.params]
            opt_params = self.master
        else:
            self.master = None
            opt_params = self.params
        fused = torch.device(self.device).type == "cuda"
        self.optimizer = torch.optim.Adam(opt_params, lr=lr, **({"fused": True} if fused else {}))
        self.step_count = 0
        self.last_loss = None

    def _skip_rng_for_layers(self, n: int) -> None:
        h, f = self.config.embedding_dim, self.config.ffn_embedding_dim
        for _ in range(n):
            for shape in ((3 * h, h), (h, h), (f, h), (h, f)):
                torch.nn.init.xavier_normal_(torch.empty(shape))

    # ---- inputs -----------------------------------------------------------------
    def create_inputs(self, step: Optional[int] = None) -> torch.Tensor:
        """Full ``[L, B, H]`` input of this data-parallel replica (same on all its ranks)."""
        g = torch.Generator().manual_seed(1000003 * (self.seed + 1) + 7919 * self.dp_idx
                                          + (self.step_count if step is None else step))
        c = self.config
        x = torch.randn(c.seq_len, c.batch_size, c.embedding_dim, generator=g)
        return x.to(self.device, self.low_dtype)

    # ---- forward ------------------------------------------------------------------
    def forward_step(self, full_input: Optional[torch.Tensor]):
        cfg = self.config
        nb, ns = len(self.batch_slices), len(self.seq_slices)
        rec = np.empty((nb, ns), dtype=object)
        if self.is_first:
            grid = grid_slice_batch_and_sequence(full_input, self.batch_slices, self.seq_slices)
        loss_sum = torch.zeros((), dtype=torch.float64)
        for bi, b in enumerate(self.batch_slices):
            cache = self.layers.create_cache(b, cfg.seq_len)
            c = 0
            for si, t in enumerate(self.seq_slices):
                t_loc = t // self.topo.tp if self.sequence_parallel else t
                if self.is_first:
                    x = grid[bi, si]
                    if self.sequence_parallel:  # my chunk of the slice's tokens
                        x = x[self.tp_idx * t_loc:(self.tp_idx + 1) * t_loc].contiguous()
                else:
                    x = torch.empty(t_loc, b, cfg.embedding_dim, device=self.device, dtype=self.low_dtype)
                    p2p.recv_forward(x)
                x.requires_grad_(True)
                h, prefixes, news = x, [], []
                for layer, (ck, cv) in zip(self.layers.layers, cache):
                    pk = ck[:, :c].detach().clone().requires_grad_() if c else None
                    pv = cv[:, :c].detach().clone().requires_grad_() if c else None
                    h, nk, nv = layer.forward_slice(h, pk, pv)
                    with torch.no_grad():
                        ck[:, c:c + t].copy_(nk)
                        cv[:, c:c + t].copy_(nv)
                    prefixes.append((pk, pv))
                    news.append((nk, nv))
                rec[bi, si] = (x, h, prefixes, news, c, t, b)
                if self.is_last:
                    loss_sum += h.detach().double().sum().cpu()
                else:
                    p2p.send_forward(h.detach())
                c += t
        if self.is_last:
            if self.sequence_parallel:  # every rank summed its token chunks only
                dist.all_reduce(loss_sum, group=mpu.get_model_parallel_group())
            self.last_loss = float(loss_sum) / (cfg.seq_len * cfg.batch_size * cfg.embedding_dim)
        return rec

    # ---- backward -----------------------------------------------------------------
    def backward_step(self, rec, output_grad=None):
        """``output_grad``: optional ``[L, B, H]`` gradient of the stage output (last stage only);
        default is the seed gradient of ``loss = mean(output)`` times the loss scale."""
        cfg = self.config
        numel = cfg.seq_len * cfg.batch_size * cfg.embedding_dim
        n_params = len(self.params)
        for bi in reversed(range(len(self.batch_slices))):
            b = self.batch_slices[bi]
            h_local = self.layers.layers[0].attn.num_heads if len(self.layers.layers) else 0
            d = cfg.attention_heads_dim
            acc = [(torch.zeros(b * h_local, cfg.seq_len, d, device=self.device),
                    torch.zeros(b * h_local, cfg.seq_len, d, device=self.device))
                   for _ in self.layers.layers]
            for si in reversed(range(len(self.seq_slices))):
                x, y, prefixes, news, c, t, _ = rec[bi, si]
                if self.is_last and output_grad is not None:
                    boff = sum(self.batch_slices[:bi])
                    r0 = c + (self.tp_idx * (t // self.topo.tp) if self.sequence_parallel else 0)
                    dy = output_grad[r0:r0 + y.shape[0], boff:boff + b].to(y.dtype).contiguous()
                elif self.is_last:
                    dy = torch.full_like(y, self.loss_scale / numel)
                else:
                    dy = torch.empty_like(y)
                    p2p.recv_backward(dy)
                outputs, grad_outputs = [y], [dy]
                for (nk, nv), (ak, av) in zip(news, acc):
                    outputs += [nk, nv]
                    grad_outputs += [ak[:, c:c + t].to(nk.dtype), av[:, c:c + t].to(nv.dtype)]
                inputs = self.params + [x]
                if c:
                    for pk, pv in prefixes:
                        inputs += [pk, pv]
                grads = torch.autograd.grad(outputs, inputs, grad_outputs, allow_unused=True)
                for g, mg in zip(grads[:n_params], self.main_grads):
                    if g is not None:
                        mg.add_(g)
                if not self.is_first:
                    p2p.send_backward(grads[n_params])
                if c:
                    rest = grads[n_params + 1:]
                    for li, (ak, av) in enumerate(acc):
                        ak[:, :c].add_(rest[2 * li])
                        av[:, :c].add_(rest[2 * li + 1])
                rec[bi, si] = None

    # ---- gradient reduction and update ---------------------------------------------
    def allreduce_params(self):
        if self._partial_grad_ids:
            flat = torch.cat([self.main_grads[i].reshape(-1) for i in self._partial_grad_ids])
            dist.all_reduce(flat, group=mpu.get_model_parallel_group())
            off = 0
            for i in self._partial_grad_ids:
                g = self.main_grads[i]
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()
        dp = self.topo.dp
        if dp == 1:
            return
        flat = torch.cat([g.reshape(-1) for g in self.main_grads])
        dist.all_reduce(flat, group=mpu.get_data_parallel_group())
        flat.div_(dp)
        off = 0
        for g in self.main_grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()

    def unscaled_grads(self) -> List[torch.Tensor]:
        return [g / self.loss_scale for g in self.main_grads]

    def update_weights(self):
        targets = self.master if self.mixed_precision else self.params
        for p, g in zip(targets, self.main_grads):
            p.grad = (g / self.loss_scale).to(p.dtype)
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        if self.mixed_precision:
            with torch.no_grad():
                for p, m in zip(self.params, self.master):
                    p.copy_(m)
        for g in self.main_grads:
            g.zero_()

    def compute_grads(self, full_input=None):
        """Forward + backward (+ DP all-reduce); leaves scaled grads in ``main_grads``."""
        for g in self.main_grads:
            g.zero_()
        if full_input is None and self.is_first:
            full_input = self.create_inputs()
        rec = self.forward_step(full_input)
        self.backward_step(rec)
        self.allreduce_params()

    def step(self, full_input=None):
        self.compute_grads(full_input)
        self.update_weights()
        self.step_count += 1
        return self.last_loss

    # ---- state ----------------------------------------------------------------------
    def named_grads(self):
        names = [n for n, _ in self.layers.named_parameters()]
        return {f"layers.{n}": g for n, g in zip(names, self.unscaled_grads())}

    def state_dict(self):
        return {f"layers.{k}": v for k, v in self.layers.state_dict().items()}

    def load_state_dict(self, sd):
        self.layers.load_state_dict({k[len("layers."):]: v for k, v in sd.items()})
        if self.mixed_precision:
            with torch.no_grad():
                for p, m in zip(self.params, self.master):
                    m.copy_(p)


def run_timed(pipeline, n_steps, warmup_steps=5, verbose=False):
    """Host-clock step times with a device drain per step (reference:
    test_transformer_terapipe.py:288-304); returns (mean, std) over post-warm-up steps."""
    times = []
    for _ in range(n_steps):
        t0 = time.time()
        pipeline.step()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        times.append(time.time() - t0)
        if verbose:
            print("rank", pipeline.rank, "step_time:", times[-1], flush=True)
    kept = times[warmup_steps:] if len(times) > warmup_steps else times
    return float(np.mean(kept)), float(np.std(kept))
