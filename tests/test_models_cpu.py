"""CPU checks of configs, slicing helpers, the portable layer and the token-slice pipeline."""
import os
import sys

import pytest
import torch

from terapipe_b200.models import (BATCH_CONFIGS, MODEL_CONFIGS, TransformerConfig, TransformerLayer,
                                  grid_slice_batch_and_sequence, merge_state_dicts,
                                  slice_state_dict, uniform_slice_layers, uniform_slice_x)
from terapipe_b200.parallel.topology import Topology
from terapipe_b200.runtime.portable import PortablePipeline
from terapipe_b200.utils import checkpoint, uniform_slice


def test_registry_matches_reference_table():
    assert len(MODEL_CONFIGS) == 35
    assert MODEL_CONFIGS["test"] == (24, 256, 128, 4)
    assert MODEL_CONFIGS["gpt3-1b"] == (24, 2048, 2048, 16)
    assert MODEL_CONFIGS["gpt3-13b"] == (40, 5120, 2048, 40)
    assert MODEL_CONFIGS["gpt3-44b"] == (96, 6144, 2048, 48)
    assert MODEL_CONFIGS["gpt3-175b"] == (96, 12288, 2048, 96)
    assert MODEL_CONFIGS["gpt3-175b-megatron"] == (48, 6144, 2048, 384)
    assert MODEL_CONFIGS["megatron-8b"] == (72, 3072, 1024, 32)
    assert MODEL_CONFIGS["gpt3-2b"] == (32, 2560, 2048, 32)
    assert BATCH_CONFIGS == {"gpt3-1b": 72, "gpt3-13b": 32, "gpt3-44b": 16, "gpt3-175b": 2,
                             "gpt3-13b-4096": 8, "gpt3-13b-6144": 4, "gpt3-13b-8192": 2}


def test_config_from_predefined_and_override():
    cfg = TransformerConfig.from_predefined_model("gpt3-175b", n_devices=8, batch_size=2, n_layers=8)
    assert (cfg.n_layers, cfg.embedding_dim, cfg.ffn_embedding_dim) == (8, 12288, 49152)
    assert cfg.attention_heads_dim == 128
    x = TransformerConfig(batch_size=2, seq_len=16, embedding_dim=64, n_devices=1).create_inputs("cpu")
    assert x.shape == (16, 2, 64)


def test_uniform_slice_and_grid():
    assert uniform_slice(10, 3) == [4, 3, 3]
    assert uniform_slice(2048, 16) == [128] * 16
    x = torch.arange(6 * 4 * 2, dtype=torch.float32).view(6, 4, 2)
    grid = grid_slice_batch_and_sequence(x, [1, 3], [2, 4])
    assert grid.shape == (2, 2)
    assert torch.equal(grid[1, 1], x[2:, 1:])
    assert grid[0, 0].is_contiguous() and not grid[0, 0].requires_grad
    with pytest.raises(AssertionError):
        grid_slice_batch_and_sequence(x, [1, 2], [2, 4])
    parts = uniform_slice_x(x, 4)
    assert [p.size(0) for p in parts] == [2, 2, 1, 1]
    assert [len(s) for s in uniform_slice_layers(list(range(10)), 4)] == [3, 3, 2, 2]


def test_topology_matches_reference_layout():
    topo = Topology(16, 4, 2)
    assert topo.dp == 2
    assert topo.tp_groups()[:2] == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert topo.dp_groups()[0] == [0, 8] and topo.dp_groups()[5] == [5, 13]
    assert topo.coords(13) == (1, 1, 1)
    assert topo.reference_stage_pairs() == [(3, 4), (11, 12)]
    assert (1, 5) in topo.stage_pairs() and (11, 15) in topo.stage_pairs()
    assert topo.tp_src_rank(6) == 4 and topo.tp_dst_rank(6) == 7
    assert topo.prev_stage_rank(2) is None and topo.next_stage_rank(2) == 6
    assert list(topo.layers_of_stage(5, 0)) == [0, 1, 2] and list(topo.layers_of_stage(5, 1)) == [3, 4]
    with pytest.raises(ValueError):
        Topology(6, 4, 1)


def _cfg(n_layers=2, activation="gelu"):
    return TransformerConfig(batch_size=2, seq_len=128, n_layers=n_layers, embedding_dim=256,
                             num_attention_heads=4, n_devices=1, activation=activation)


def test_sliced_matches_unsliced_fp32():
    """2 layers, hidden 256, 4 heads, GeLU, seq 128, batch 2: loss and every parameter gradient
    of 8 uniform token slices (with cached prefix KV) equal the unsliced run to 1e-5."""
    cfg = _cfg()
    ref = PortablePipeline(cfg, [2], [128], device="cpu")
    x = ref.create_inputs(0)
    ref.compute_grads(x)
    for batch_slices, seq_slices in (([2], uniform_slice(128, 8)), ([1, 1], [40, 8, 16, 64])):
        p = PortablePipeline(cfg, batch_slices, seq_slices, device="cpu")
        p.compute_grads(x)
        assert abs(p.last_loss - ref.last_loss) < 1e-5
        for a, b in zip(ref.main_grads, p.main_grads):
            assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)


def test_step_updates_and_recompute_flag():
    cfg = _cfg(n_layers=1)
    a = PortablePipeline(cfg, [2], [64, 64], device="cpu", lr=1e-3)
    b = PortablePipeline(cfg, [2], [64, 64], device="cpu", lr=1e-3, checkpoint_gradients=True)
    x = a.create_inputs(0)
    a.compute_grads(x)
    b.compute_grads(x)
    for ga, gb in zip(a.main_grads, b.main_grads):
        assert torch.allclose(ga, gb, atol=1e-6)
    before = [p.detach().clone() for p in a.params]
    a.update_weights()
    assert any(not torch.equal(p0, p1) for p0, p1 in zip(before, a.params))
    assert all(float(g.abs().max()) == 0.0 for g in a.main_grads)


def test_layer_reference_style_call_matches_slice_call():
    torch.manual_seed(0)
    layer = TransformerLayer(64, 256, 2)
    x = torch.randn(12, 3, 64)
    cache = layer.attn.create_attn_cache(3, 12, "cpu")
    y_full, _ = layer(x, None, 0)
    y0, kv0 = layer(x[:5], cache, 0)
    y1, kv1 = layer(x[5:], cache, 5)
    assert torch.allclose(torch.cat([y0, y1]), y_full, atol=1e-5)
    assert kv1[0].shape == (3 * 2, 12, 32)


def test_checkpoint_function_contract():
    w = torch.randn(4, 4, requires_grad=True)
    x = torch.randn(3, 4, requires_grad=True)

    def fn(a):
        return torch.tanh(a @ w)

    y = checkpoint.CheckpointFunction.apply(fn, 1, x, w)
    gx, gw = torch.autograd.grad(y.sum(), [x, w])
    y2 = fn(x)
    gx2, gw2 = torch.autograd.grad(y2.sum(), [x, w])
    assert torch.allclose(gx, gx2) and torch.allclose(gw, gw2)


def test_slice_state_dict_roundtrip():
    cfg = _cfg(n_layers=3)
    p = PortablePipeline(cfg, [2], [128], device="cpu")
    full = {"layers." + k: v for k, v in p.layers.state_dict().items()}
    shards = {(s, r): slice_state_dict(3, full, tp=2, tp_rank=r, pp=2, pp_rank=s)
              for s in range(2) for r in range(2)}
    assert shards[(0, 0)]["layers.layers.0.attn.in_proj.weight"].shape == (384, 256)
    assert shards[(1, 1)]["layers.layers.0.fc2.weight"].shape == (256, 512)
    assert "layers.layers.1.fc1.bias" in shards[(0, 0)] and "layers.layers.1.fc1.bias" not in shards[(1, 0)]
    merged = merge_state_dicts(3, shards, tp=2, pp=2)
    assert set(merged) == set(full)
    for k in full:
        assert torch.equal(merged[k], full[k]), k


REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "transformer_models.py")),
                    reason="reference not installed under baseline/_ref")
def test_relu_layer_matches_reference_layer():
    """Same weights, ReLU mode: our layer equals the reference's ModelParallelTransformerLayer."""
    import subprocess
    code = r'''
import sys, torch
sys.path.insert(0, %r)
import torch.distributed as dist
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29611", rank=0, world_size=1)
import mpu
mpu.initialize_model_parallel(1, 1)
from transformer_models import ModelParallelTransformerLayer as RefLayer
torch.manual_seed(0)
ref = RefLayer(64, 256, 2, device="cpu")
torch.manual_seed(1)
x = torch.randn(10, 2, 64)
k, v = ref.attn.create_attn_cache(2, 10, device="cpu")
y0, c0 = ref(x[:4].clone(), (k, v), 0)
y1, c1 = ref(x[4:].clone(), c0, 4)
torch.save({"sd": ref.state_dict(), "x": x, "y": torch.cat([y0, y1]).detach()}, sys.argv[1])
''' % REF
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "ref.pt")
        subprocess.run([sys.executable, "-c", code, out], check=True, timeout=120,
                       env={**os.environ, "PYTHONPATH": ""})
        blob = torch.load(out)
    mine = TransformerLayer(64, 256, 2, activation="relu")
    mine.load_state_dict(blob["sd"])
    cache = mine.attn.create_attn_cache(2, 10, "cpu")
    y0, _ = mine(blob["x"][:4], cache, 0)
    y1, _ = mine(blob["x"][4:], cache, 4)
    assert torch.allclose(torch.cat([y0, y1]), blob["y"], atol=1e-5)


def test_assign_cache_appends_in_place_and_routes_gradients():
    """KV-append op of the reference API (transformer_models.py:177-193)."""
    from transformer_models import assign_cache_
    torch.manual_seed(0)
    k1 = torch.randn(2, 3, 4, requires_grad=True)
    k2 = torch.randn(2, 5, 4, requires_grad=True)
    w = torch.randn(2, 8, 4)
    cache = torch.zeros(2, 8, 4).requires_grad_()
    c = assign_cache_(cache, k1, (slice(None), slice(0, 3)))
    used_early = (c[:, :3] * w[:, :3]).sum()          # a consumer between the two appends
    c = assign_cache_(c, k2, (slice(None), slice(3, 8)))
    (used_early + (c * w).sum()).backward()
    assert torch.equal(cache.data[:, :3], k1.data) and torch.equal(cache.data[:, 3:], k2.data)
    assert torch.allclose(k1.grad, 2 * w[:, :3])      # seen by both consumers
    assert torch.allclose(k2.grad, w[:, 3:])


def test_terapipe_backward_hook_replays_slices_in_reverse():
    """Reference API for user-written sliced forwards (terapipe.py:154-214): a toy layer whose
    slice j reads a running 'cache' (prefix sums) produced by the earlier slices."""
    import numpy as np
    from terapipe import loss_func, terapipe_backward_hook
    from transformer_models import grid_slice_batch_and_sequence
    torch.manual_seed(0)
    L, B, H = 8, 2, 3
    w = torch.randn(H, H, requires_grad=True)
    x = torch.randn(L, B, H)

    def whole(xx):  # y_t = (x_t + sum_{s<t} x_s @ w) @ w
        prefix = torch.cumsum(xx @ w, 0) - xx @ w
        return (xx + prefix) @ w

    ref_loss = loss_func(whole(x))
    ref_loss.backward()
    ref_grad, w.grad = w.grad.clone(), None

    batch_slices, seq_slices = [1, 1], [3, 5]
    xs = grid_slice_batch_and_sequence(x, batch_slices, seq_slices)
    shape = (len(batch_slices), len(seq_slices))
    outputs, cache_in, cache_out = (np.empty(shape, dtype=object) for _ in range(3))
    for i in range(shape[0]):
        carry = torch.zeros(xs[i, 0].shape[1], H)          # sum of x_s @ w over earlier slices
        for j in range(shape[1]):
            c_in = carry.detach().requires_grad_()
            proj = xs[i, j] @ w
            prefix = torch.cumsum(proj, 0) - proj + c_in
            outputs[i, j] = (xs[i, j] + prefix) @ w
            carry = c_in + proj.sum(0)
            cache_in[i, j], cache_out[i, j] = [c_in], [carry]
    y = terapipe_backward_hook(outputs, cache_in, cache_out, batch_slices, seq_slices, cat_outputs=True)
    loss = loss_func(y)
    loss.backward()
    assert torch.allclose(loss, ref_loss, atol=1e-6)
    assert torch.allclose(w.grad, ref_grad, atol=1e-5)


def test_module_style_helpers_exist_and_build_a_stage():
    """initialize_model / LOSS_SCALE_FACTOR of the module-style driver (terapipe.py:30,274-288)."""
    import argparse
    import terapipe as tpipe
    assert tpipe.LOSS_SCALE_FACTOR == 128.0
    args = argparse.Namespace(model="test", batch_size=2, n_batch_slices=1, n_input_slices=4,
                              mixed_precision=False, world_size=1, n_layers=2)
    config, layers, pipelined = tpipe.initialize_model(args)
    assert config.n_total_layers == 2 and config.n_layers == 2
    y = pipelined(torch.randn(config.seq_len, 2, config.embedding_dim))
    tpipe.loss_func(y).backward()
    assert all(p.grad is not None for p in pipelined.parameters())


def test_assign_cache_backward_leaves_the_incoming_gradient_untouched():
    """Autograd may hand backward a tensor the caller still owns (``grad_outputs``): the KV-append
    op must build the earlier cache's gradient in a new tensor."""
    import torch
    from terapipe_b200.models.layers import assign_cache_
    cache = torch.zeros(2, 6, 3, requires_grad=True)
    value = torch.randn(2, 2, 3, requires_grad=True)
    idx = (slice(None), slice(2, 4))
    out = assign_cache_(cache, value, idx)
    g = torch.randn(2, 6, 3)
    g_before = g.clone()
    g_cache, g_value = torch.autograd.grad(out, [cache, value], grad_outputs=g)
    assert torch.equal(g, g_before)
    assert torch.equal(g_value, g_before[idx])
    assert torch.equal(g_cache[idx], torch.zeros(2, 2, 3))
    keep = torch.ones(6, dtype=torch.bool)
    keep[2:4] = False
    assert torch.equal(g_cache[:, keep], g_before[:, keep])


def test_head_padding_keeps_attention_and_gradients():
    """The engine's zero-padding of heads (80 -> 128 columns): padded projections with the
    softmax scale of the real width give the same attention output and the same gradients for
    the real entries, zero gradients for the padding, and pad / unpad are inverse."""
    import types

    from terapipe_b200.runtime.engine import StageEngine
    h, D, Dk, H, T = 2, 80, 128, 160, 12
    eng = types.SimpleNamespace(h=h, D=D, Dk=Dk, Hl=h * Dk, _HEAD_PADDED=StageEngine._HEAD_PADDED)
    pad = lambda n, w: StageEngine._pad_heads(eng, n, w)
    unpad = lambda n, w: StageEngine._unpad_heads(eng, n, w)
    g = torch.Generator().manual_seed(0)
    w_in = torch.randn(3 * h * D, H, generator=g, dtype=torch.float64) / 8
    b_in = torch.randn(3 * h * D, generator=g, dtype=torch.float64)
    w_out = torch.randn(H, h * D, generator=g, dtype=torch.float64) / 8
    x = torch.randn(T, H, generator=g, dtype=torch.float64)
    for n, w in (("attn.in_proj.weight", w_in), ("attn.in_proj.bias", b_in), ("attn.out_proj.weight", w_out)):
        assert torch.equal(unpad(n, pad(n, w)), w)
    assert torch.equal(pad("fc1.weight", w_in), w_in)

    def attention(wi, bi, wo, d):
        qkv = (x @ wi.t() + bi).view(T, h, 3, d)
        q, k, v = (qkv[:, :, i].transpose(0, 1) for i in range(3))
        s = (q @ k.transpose(1, 2)) * D ** -0.5
        s = s.masked_fill(torch.ones(T, T).triu(1).bool(), float("-inf"))
        o = (s.softmax(-1) @ v).transpose(0, 1).reshape(T, h * d)
        return o @ wo.t()

    plain = [t.clone().requires_grad_() for t in (w_in, b_in, w_out)]
    padded = [pad(n, t).clone().requires_grad_() for n, t in
              (("attn.in_proj.weight", w_in), ("attn.in_proj.bias", b_in), ("attn.out_proj.weight", w_out))]
    y0, y1 = attention(*plain, D), attention(*padded, Dk)
    assert torch.allclose(y0, y1, atol=1e-12)
    y0.square().sum().backward()
    y1.square().sum().backward()
    for n, a, b in zip(("attn.in_proj.weight", "attn.in_proj.bias", "attn.out_proj.weight"), plain, padded):
        assert torch.allclose(unpad(n, b.grad), a.grad, atol=1e-10), n
        assert torch.equal(pad(n, unpad(n, b.grad)), b.grad), n    # the padding's gradient is zero
