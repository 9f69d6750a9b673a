"""Multi-process (gloo, CPU) checks: group construction, tensor + pipeline + data parallel
equivalence with the single-rank unsliced run, mpu layers, and host-side failure detection."""
import pytest
import torch

from dist_utils import run_ranks


def _cfg(n_layers=4):
    from terapipe_b200.models import TransformerConfig
    return TransformerConfig(batch_size=2, seq_len=64, n_layers=n_layers, embedding_dim=64,
                             num_attention_heads=4, n_devices=1)


def _single_rank_reference(n_layers=4, batch=2):
    from terapipe_b200.runtime.portable import PortablePipeline
    cfg = _cfg(n_layers)
    cfg.batch_size = batch
    p = PortablePipeline(cfg, [batch], [64], device="cpu")
    x = p.create_inputs(0)
    p.compute_grads(x)
    return p.last_loss, p.named_grads(), x


def _rank_pipeline(rank, world, tp, pp, batch_slices, seq_slices, sequence_parallel=False):
    from terapipe_b200 import parallel as mpu
    from terapipe_b200.runtime.portable import PortablePipeline
    mpu.initialize_model_parallel(tp, pp, verbose=False)
    topo = mpu.get_topology()
    cfg = _cfg()
    p = PortablePipeline(cfg, batch_slices, seq_slices, device="cpu", sequence_parallel=sequence_parallel)
    x = p.create_inputs(0) if p.is_first else None
    p.compute_grads(x)
    out = {"coords": topo.coords(rank), "loss": p.last_loss, "grads": p.named_grads(),
           "layer_ids": list(p.layer_ids),
           "groups": (mpu.get_model_parallel_rank(), mpu.get_pipeline_parallel_group_rank(),
                      mpu.get_data_parallel_rank(), mpu.get_model_parallel_src_rank(),
                      mpu.get_model_parallel_dst_rank())}
    mpu.destroy_model_parallel()
    return out


@pytest.mark.parametrize("tp,pp,world", [(2, 2, 4), (1, 2, 2), (2, 1, 2), (1, 2, 4)])
def test_parallel_layouts_match_single_rank(tp, pp, world):
    from terapipe_b200.models import slice_state_dict
    loss, full_grads, _ = _single_rank_reference()
    results = run_ranks(_rank_pipeline, world, tp, pp, [1, 1], [8, 24, 16, 16])
    for rank, res in enumerate(results):
        dp_idx, pp_idx, tp_idx = res["coords"]
        assert res["groups"][:3] == (tp_idx, pp_idx, dp_idx)
        if pp_idx == pp - 1:
            assert abs(res["loss"] - loss) < 1e-5 or world // (tp * pp) > 1
        want = slice_state_dict(4, full_grads, tp=tp, tp_rank=tp_idx, pp=pp, pp_rank=pp_idx)
        assert set(want) == set(res["grads"])
        if world // (tp * pp) == 1:   # with DP replicas the inputs differ per replica
            for k, g in want.items():
                assert torch.allclose(res["grads"][k], g, atol=2e-6, rtol=1e-4), (rank, k)


@pytest.mark.parametrize("tp,pp,world", [(2, 1, 2), (2, 2, 4)])
def test_sequence_parallel_pipeline_matches_single_rank(tp, pp, world):
    """Token-sharded activations between the GEMM pairs and on the pipeline links."""
    from terapipe_b200.models import slice_state_dict
    loss, full_grads, _ = _single_rank_reference()
    results = run_ranks(_rank_pipeline, world, tp, pp, [1, 1], [8, 24, 16, 16], True)
    for rank, res in enumerate(results):
        _, pp_idx, tp_idx = res["coords"]
        if pp_idx == pp - 1:
            assert abs(res["loss"] - loss) < 1e-5
        want = slice_state_dict(4, full_grads, tp=tp, tp_rank=tp_idx, pp=pp, pp_rank=pp_idx)
        for k, g in want.items():
            assert torch.allclose(res["grads"][k], g, atol=2e-6, rtol=1e-4), (rank, k)


def _rank_dp(rank, world):
    from terapipe_b200 import parallel as mpu
    from terapipe_b200.runtime.portable import PortablePipeline
    mpu.initialize_model_parallel(1, 1, verbose=False)
    cfg = _cfg(2)
    cfg.batch_size = 1
    p = PortablePipeline(cfg, [1], [32, 32], device="cpu")
    x = p.create_inputs(0)
    p.compute_grads(x)
    return {"x": x, "grads": p.named_grads()}


def test_data_parallel_averages_replica_gradients():
    from terapipe_b200.runtime.portable import PortablePipeline
    results = run_ranks(_rank_dp, 2)
    assert not torch.equal(results[0]["x"], results[1]["x"])     # each replica has its own input
    cfg = _cfg(2)
    cfg.batch_size = 1
    grads = []
    for r in range(2):
        p = PortablePipeline(cfg, [1], [64], device="cpu")
        p.compute_grads(results[r]["x"])
        grads.append(p.named_grads())
    for k in grads[0]:
        # each replica's loss is the mean over ITS batch; DP averages the two
        mean = (grads[0][k] + grads[1][k]) / 2
        assert torch.allclose(results[0]["grads"][k], mean, atol=2e-6, rtol=1e-4), k
        assert torch.equal(results[0]["grads"][k], results[1]["grads"][k])


def _rank_mpu_layers(rank, world):
    import torch.nn.functional as F
    from terapipe_b200 import parallel as mpu
    mpu.initialize_model_parallel(world, 1, verbose=False)
    torch.manual_seed(0)
    col = mpu.ColumnParallelLinear(16, 24, gather_output=True, keep_master_weight_for_test=True)
    row = mpu.RowParallelLinear(24, 8, input_is_parallel=False, keep_master_weight_for_test=True)
    emb = mpu.VocabParallelEmbedding(32, 16)
    pemb = mpu.ParallelEmbedding(32, 16)
    torch.manual_seed(1)
    x = torch.randn(5, 16, requires_grad=True)
    y = row(col(x))
    ref = F.linear(F.linear(x, col.master_weight), row.master_weight)
    y.sum().backward()
    ids = torch.tensor([[0, 5, 31], [17, 16, 15]])
    logits = torch.randn(4, 32 // world)
    target = torch.tensor([0, 31, 16, 7])
    ce = mpu.vocab_parallel_cross_entropy(logits.clone().requires_grad_(), target)
    gathered = mpu.gather_from_model_parallel_region(logits)
    ce_ref = torch.nn.functional.cross_entropy(gathered, target, reduction="none")
    data = mpu.broadcast_data(["a", "b"], {"a": torch.arange(6).view(2, 3) + 10 * rank,
                                           "b": torch.arange(4) + 100 * rank}, torch.int64)
    mpu.model_parallel_cuda_manual_seed(1234)
    with mpu.get_cuda_rng_tracker().fork():
        r_mp = torch.rand(1).item()
    r_default = torch.rand(1).item()
    return {"y_err": (y - ref).abs().max().item(), "x_grad": x.grad.clone(),
            "emb": emb(ids).detach(), "pemb_shape": tuple(pemb(ids).shape),
            "ce_err": (ce - ce_ref).abs().max().item(), "data": data,
            "r_mp": r_mp, "r_default": r_default, "split": mpu.divide(24, world)}


def test_mpu_layers_two_ranks():
    res = run_ranks(_rank_mpu_layers, 2)
    for r in res:
        assert r["y_err"] < 1e-5 and r["ce_err"] < 1e-5
        assert r["pemb_shape"] == (2, 3, 16) and r["split"] == 12
        assert torch.equal(r["data"]["a"], torch.arange(6).view(2, 3))      # rank 0's payload
        assert torch.equal(r["data"]["b"], torch.arange(4))
    assert torch.allclose(res[0]["x_grad"], res[1]["x_grad"])
    assert torch.allclose(res[0]["emb"], res[1]["emb"])
    assert res[0]["r_mp"] != res[1]["r_mp"]              # sharded-region stream differs per TP rank
    assert res[0]["r_default"] == res[1]["r_default"]    # replicated-region stream is shared


def _rank_verify(rank, world, path, mode):
    from terapipe_b200.runtime import verify
    return verify.verify_one_step(path, mode, model="test", n_layers=2, batch_size=2,
                                  tp=1 if mode == "save" else 2, pp=1 if mode == "save" else 2,
                                  n_batch_slices=1 if mode == "save" else 2,
                                  n_input_slices=1 if mode == "save" else 4, device="cpu")


def test_verify_save_then_load_across_layouts(tmp_path):
    run_ranks(_rank_verify, 1, str(tmp_path), "save")
    for name in ("input.pt", "model.ckpt", "model.grad.ckpt"):
        assert (tmp_path / name).exists()
    results = run_ranks(_rank_verify, 4, str(tmp_path), "load")
    assert all(r["ok"] for r in results)


# ---------------------------------------------------------------- failure detection (host side)
def _rank_dies(rank, world):
    from terapipe_b200 import parallel as mpu
    from terapipe_b200.runtime.portable import PortablePipeline
    mpu.initialize_model_parallel(1, 2, verbose=False)
    p = PortablePipeline(_cfg(2), [2], [32, 32], device="cpu")
    if rank == 1:
        raise RuntimeError("injected failure on the last stage before its first receive")
    p.compute_grads(p.create_inputs(0))
    return "unreachable"


def test_surviving_rank_raises_when_peer_dies():
    errors = run_ranks(_rank_dies, 2, timeout_s=20, expect_failure=True)
    assert 1 in errors and "injected failure" in errors[1]
    assert 0 in errors          # the sender's p2p call fails or times out instead of hanging


def _rank_sequence_parallel(rank, world):
    """Column/Row parallel pair on token-sharded activations against the unsharded product."""
    import torch.nn.functional as F
    from terapipe_b200 import parallel as mpu
    mpu.initialize_model_parallel(world, 1, verbose=False)
    torch.manual_seed(0)
    col = mpu.ColumnParallelLinear(16, 24, gather_output=False, keep_master_weight_for_test=True,
                                   sequence_parallel=True)
    row = mpu.RowParallelLinear(24, 16, input_is_parallel=True, keep_master_weight_for_test=True,
                                sequence_parallel=True)
    torch.manual_seed(1)
    x_full = torch.randn(8, 3, 16)                       # [tokens, batch, hidden], replicated
    x_full.requires_grad_()
    x_loc = mpu.scatter_to_sequence_parallel_region(x_full)          # my tokens
    y_loc = row(torch.relu(col(x_loc)))                              # my tokens of the output
    y = mpu.gather_from_sequence_parallel_region(y_loc, tensor_parallel_output_grad=False)
    w = torch.arange(y.numel(), dtype=torch.float32).view_as(y) / y.numel()
    (y * w).sum().backward()
    xr = x_full.detach().clone().requires_grad_()
    ref = F.linear(torch.relu(F.linear(xr, col.master_weight)), row.master_weight)
    (ref * w).sum().backward()
    return {"y_err": (y - ref).abs().max().item(), "dx_err": (x_full.grad - xr.grad).abs().max().item(),
            "loc_tokens": x_loc.shape[0], "y_loc_tokens": y_loc.shape[0]}


def test_sequence_parallel_mappings_two_ranks():
    for r in run_ranks(_rank_sequence_parallel, 2):
        assert r["loc_tokens"] == 4 and r["y_loc_tokens"] == 4
        assert r["y_err"] < 1e-5
        # every rank holds the full input gradient after the backward all-gather of the scatter
        assert r["dx_err"] < 1e-5


def _rank_sequence_parallel_layer(rank, world):
    """A layer on token-sharded activations (two slices with a KV prefix) against the same layer
    with replicated activations."""
    from terapipe_b200 import parallel as mpu
    from terapipe_b200.models import TransformerLayer
    mpu.initialize_model_parallel(world, 1, verbose=False)
    out = {}
    for sp in (False, True):
        torch.manual_seed(0)
        layer = TransformerLayer(32, 128, 4, sequence_parallel=sp)
        torch.manual_seed(1)
        x = torch.randn(12, 2, 32)
        slices = [x[:8].clone().requires_grad_(), x[8:].clone().requires_grad_()]
        ys, pk, pv = [], None, None
        for xs in slices:
            inp = mpu.scatter_to_sequence_parallel_region(xs) if sp else xs
            y, nk, nv = layer.forward_slice(inp, pk, pv)
            if sp:
                y = mpu.gather_from_sequence_parallel_region(y, tensor_parallel_output_grad=False)
            ys.append(y)
            pk = nk if pk is None else torch.cat([pk, nk], 1)
            pv = nv if pv is None else torch.cat([pv, nv], 1)
        y = torch.cat(ys, 0)
        (y * torch.linspace(0, 1, y.numel()).view_as(y)).sum().backward()
        layer.allreduce_sequence_parallel_grads()
        out[sp] = {"y": y.detach(), "dx": torch.cat([s.grad for s in slices], 0),
                   "grads": {k: p.grad.clone() for k, p in layer.named_parameters()}}
    return out


def test_sequence_parallel_layer_matches_replicated_layer():
    for r in run_ranks(_rank_sequence_parallel_layer, 2):
        assert torch.allclose(r[True]["y"], r[False]["y"], atol=1e-5)
        assert torch.allclose(r[True]["dx"], r[False]["dx"], atol=1e-5)
        for k, g in r[False]["grads"].items():
            assert torch.allclose(r[True]["grads"][k], g, atol=2e-5), k
