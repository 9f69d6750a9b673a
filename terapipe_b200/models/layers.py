"""Portable (pure torch) pre-LN Transformer layer for one token slice.

Math of the reference layer (transformer_models.py:196-327):

* ``in_proj`` output columns are per-head interleaved: head ``i`` owns columns
  ``[3d*i, 3d*(i+1))`` = (q, k, v); tensor-parallel shards are contiguous head groups.
* ``q`` is scaled by ``d**-0.5``; the slice's ``t`` queries attend to ``c`` cached
  prefix positions plus themselves under a causal mask (additive ``-65504`` above the
  diagonal of the last ``t`` columns); softmax runs in fp32.
* ``x = x + attn(LN(x))``, ``x = x + fc2(act(fc1(LN(x))))``; no dropout.

This module is the CPU/gloo path and the numerical oracle for the sm_100a engine.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .. import parallel as mpu
from ..utils import checkpoint as ckpt
from .config import NEG_INF


class _AssignCache(torch.autograd.Function):
    """KV-append: write ``value`` into ``cache[index]`` in place and return ``cache``
    (reference: transformer_models.py:177-193).  The gradient of the written region flows to
    ``value``; the rest flows to the earlier cache.  Backward never writes into the incoming
    gradient (autograd may hand over a caller's ``grad_outputs`` tensor or a retained ``.grad``):
    the gradient of the earlier cache is a new tensor with the slice zeroed."""

    @staticmethod
    def forward(ctx, cache, value, index):
        ctx.index = index
        cache.data[index] = value  # through .data: the version counter must not move
        return cache

    @staticmethod
    def backward(ctx, grad_cache_output):
        grad_value = grad_cache_output[ctx.index].clone()
        grad_cache = grad_cache_output.clone()
        grad_cache[ctx.index] = 0
        return grad_cache, grad_value, None


assign_cache_ = _AssignCache.apply


class MultiheadLMAttentionWithCache(nn.Module):
    def __init__(self, embed_dim, num_heads, bias=True, device="cpu", sequence_parallel=False):
        super().__init__()
        tp = mpu.get_model_parallel_world_size()
        if num_heads % tp or embed_dim % num_heads:
            raise AssertionError("heads must divide the width and the tensor-parallel size the heads")
        self.embed_dim = embed_dim
        self.num_total_heads = num_heads
        self.num_heads = num_heads // tp
        self.head_dim = embed_dim // num_heads
        self.scaling = self.head_dim ** -0.5
        self.model_parallel_size = tp
        # sequence_parallel: input and output hold this rank's chunk of the slice's tokens; the
        # projections all-gather / reduce-scatter over the tensor-parallel group
        self.in_proj = mpu.ColumnParallelLinear(embed_dim, 3 * embed_dim, bias=bias,
                                                gather_output=False, device=device,
                                                sequence_parallel=sequence_parallel)
        self.out_proj = mpu.RowParallelLinear(embed_dim, embed_dim, bias=bias,
                                              input_is_parallel=True, device=device,
                                              sequence_parallel=sequence_parallel)

    # -- building blocks ---------------------------------------------------------
    def project_qkv(self, x):
        """``x [t, b, H]`` -> ``q, k, v`` each ``[b*h, t, d]`` (q already scaled)."""
        qkv = self.in_proj(x)                      # all tokens of the slice, this rank's heads
        t, b = qkv.shape[0], qkv.shape[1]
        qkv = qkv.view(t, b * self.num_heads, 3 * self.head_dim).transpose(0, 1)
        q, k, v = qkv.chunk(3, dim=-1)
        return q * self.scaling, k, v

    @staticmethod
    def _core(q, k, v, prefix_len):
        """Scores over ``[prefix | slice]`` keys, fp32 softmax, weighted values."""
        t = q.size(1)
        scores = torch.bmm(q, k.transpose(1, 2))
        mask = scores.new_full((t, t), NEG_INF).triu_(1)
        if prefix_len:
            mask = torch.cat([scores.new_zeros(t, prefix_len), mask], dim=1)
        probs = F.softmax(scores + mask, dim=-1, dtype=torch.float32).type_as(scores)
        ctx = torch.bmm(probs, v)                       # [b*h, t, d]
        return ctx.transpose(0, 1).contiguous()         # [t, b*h, d]

    def attend(self, q, k_all, v_all, prefix_len, checkpoint_gradients=False):
        t = q.size(1)
        if checkpoint_gradients:
            fn = lambda a, b_, c_: self._core(a, b_, c_, prefix_len)  # noqa: E731
            ctx = ckpt.CheckpointFunction.apply(fn, 3, q, k_all, v_all)
        else:
            ctx = self._core(q, k_all, v_all, prefix_len)
        bsz = q.size(0) // self.num_heads
        return ctx.view(t, bsz, self.num_heads * self.head_dim)

    def forward_slice(self, x, prefix_k=None, prefix_v=None, checkpoint_gradients=False):
        """One token slice.  ``prefix_*`` are ``[b*h, c, d]`` (or None when ``c == 0``).
        Returns ``(out [t,b,H], new_k, new_v)``; the caller appends new_k/new_v to its cache."""
        q, new_k, new_v = self.project_qkv(x)
        c = 0 if prefix_k is None else prefix_k.size(1)
        k_all = new_k if c == 0 else torch.cat([prefix_k, new_k], dim=1)
        v_all = new_v if c == 0 else torch.cat([prefix_v, new_v], dim=1)
        ctx = self.attend(q, k_all, v_all, c, checkpoint_gradients)
        return self.out_proj(ctx), new_k, new_v

    def forward(self, x, full_cache=None, cache_len=0, checkpoint_gradients=False):
        """Reference-style call: ``full_cache = (k, v)`` of shape ``[b*h, L, d]`` whose
        rows ``[cache_len, cache_len+t)`` are overwritten with this slice's keys/values.
        Returns ``(out, (k_seen, v_seen))`` where ``*_seen`` cover rows ``[0, cache_len+t)``
        and carry gradients to both the prefix and the new rows."""
        if full_cache is None:
            if cache_len != 0:
                raise AssertionError("a prefix needs a cache")
            out, _, _ = self.forward_slice(x, None, None, checkpoint_gradients)
            return out, None
        cache_k, cache_v = full_cache
        t = x.size(0)
        pk = cache_k[:, :cache_len] if cache_len else None
        pv = cache_v[:, :cache_len] if cache_len else None
        out, new_k, new_v = self.forward_slice(x, pk, pv, checkpoint_gradients)
        with torch.no_grad():
            cache_k[:, cache_len:cache_len + t].copy_(new_k)
            cache_v[:, cache_len:cache_len + t].copy_(new_v)
        k_seen = new_k if pk is None else torch.cat([pk, new_k], dim=1)
        v_seen = new_v if pv is None else torch.cat([pv, new_v], dim=1)
        return out, (k_seen, v_seen)

    def create_attn_cache(self, batch_size, seq_len, device=None, dtype=torch.float32):
        device = device if device is not None else self.in_proj.weight.device
        shape = (batch_size * self.num_heads, seq_len, self.head_dim)
        return (torch.zeros(shape, device=device, dtype=dtype),
                torch.zeros(shape, device=device, dtype=dtype))


ModelParallelMultiheadLMAttentionWithCache = MultiheadLMAttentionWithCache


class TransformerLayer(nn.Module):
    """``attn_ln, attn, fc_ln, fc1, fc2`` — parameter names and shapes of the
    reference's ModelParallelTransformerLayer (transformer_models.py:314-327)."""

    def __init__(self, embedding_dim, ffn_embedding_dim, num_attention_heads, device="cpu",
                 checkpoint_gradients=False, activation="gelu", sequence_parallel=False):
        super().__init__()
        tp = mpu.get_model_parallel_world_size()
        if ffn_embedding_dim % tp:
            raise AssertionError("FFN width must be divisible by the tensor-parallel size")
        self.model_parallel_size = tp
        self.checkpoint_gradients = checkpoint_gradients
        self.activation = activation
        # sequence_parallel: the layer's input and output, both LayerNorms and the residual adds
        # work on this rank's chunk of the slice's tokens (1/tp of the activation memory and
        # LayerNorm work); the replicated parameters then receive partial gradients, see
        # allreduce_sequence_parallel_grads
        self.sequence_parallel = sequence_parallel and tp > 1
        self.attn_ln = nn.LayerNorm(embedding_dim).to(device)
        self.attn = MultiheadLMAttentionWithCache(embedding_dim, num_attention_heads, device=device,
                                                  sequence_parallel=self.sequence_parallel)
        self.fc_ln = nn.LayerNorm(embedding_dim).to(device)
        self.fc1 = mpu.ColumnParallelLinear(embedding_dim, ffn_embedding_dim,
                                            gather_output=False, device=device,
                                            sequence_parallel=self.sequence_parallel)
        self.fc2 = mpu.RowParallelLinear(ffn_embedding_dim, embedding_dim,
                                         input_is_parallel=True, device=device,
                                         sequence_parallel=self.sequence_parallel)

    def _act(self, z):
        return F.gelu(z) if self.activation == "gelu" else F.relu(z)

    def _ffn(self, x):
        return x + self.fc2(self._act(self.fc1(self.fc_ln(x))))

    def forward_slice(self, x, prefix_k=None, prefix_v=None):
        a, new_k, new_v = self.attn.forward_slice(self.attn_ln(x), prefix_k, prefix_v,
                                                  self.checkpoint_gradients)
        return self._ffn(x + a), new_k, new_v

    def forward(self, x, full_cache=None, cache_len=0):
        a, cache = self.attn(self.attn_ln(x), full_cache, cache_len,
                             checkpoint_gradients=self.checkpoint_gradients)
        return self._ffn(x + a), cache


    def allreduce_sequence_parallel_grads(self):
        """With ``sequence_parallel`` every rank sees only its tokens, so the gradients of the
        parameters that are replicated over the tensor-parallel group (LayerNorm weights and
        biases, the biases of the row-parallel projections) are partial: sum them."""
        if not self.sequence_parallel:
            return
        import torch.distributed as dist
        group = mpu.get_model_parallel_group()
        for p in (*self.attn_ln.parameters(), *self.fc_ln.parameters(), self.attn.out_proj.bias,
                  self.fc2.bias):
            if p is not None and p.grad is not None:
                dist.all_reduce(p.grad, group=group)


ModelParallelTransformerLayer = TransformerLayer


class SingleDeviceTransformer(nn.Module):
    """A plain stack of layers run on whole sequences (no slicing)."""

    def __init__(self, transformer_layers):
        super().__init__()
        self.layers = nn.ModuleList(transformer_layers)

    def forward(self, x, attn_caches=None):
        caches = attn_caches if attn_caches is not None else [None] * len(self.layers)
        new_caches = []
        for layer, cache in zip(self.layers, caches):
            x, new_cache = layer(x, cache)
            new_caches.append(new_cache)
        return x, new_caches
