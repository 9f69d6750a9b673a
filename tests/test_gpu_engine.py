"""The sm_100a engine against the portable autograd pipeline (fp32) on the same weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _oracle(cfg, x):
    from terapipe_b200.runtime.portable import PortablePipeline
    p = PortablePipeline(cfg, [cfg.batch_size], [cfg.seq_len], device="cuda")
    p.compute_grads(x.float())
    return p


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("activation", ["gelu", "relu"])
@pytest.mark.parametrize("batch_slices,seq_slices", [([2], [128]), ([2], [16] * 8),
                                                     ([1, 1], [40, 8, 16, 64])])
def test_engine_matches_portable_oracle(dtype, activation, batch_slices, seq_slices):
    from terapipe_b200.models import TransformerConfig
    from terapipe_b200.runtime.engine import StageEngine
    cfg = TransformerConfig(batch_size=2, seq_len=128, n_layers=2, embedding_dim=256,
                            num_attention_heads=4, n_devices=1, activation=activation)
    g = torch.Generator().manual_seed(123)
    x = torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g).cuda()
    oracle = _oracle(cfg, x)
    eng = StageEngine(cfg, batch_slices, seq_slices, dtype=dtype, init="reference", use_graph=False)
    # same weights (the oracle draws from the same seeded CPU generator)
    for (name, a), b in zip(eng.state_dict().items(), oracle.layers.state_dict().values()):
        assert _rel(a, b) < 5e-3, name
    eng.set_input(x)
    eng.compute_grads()
    eng.check_status()
    tol = 2e-2 if dtype == torch.float16 else 6e-2
    assert abs(eng.loss().item() - oracle.last_loss) < 2e-3
    assert _rel(eng.output(), oracle_output(oracle, x)) < tol
    want = oracle.named_grads()
    got = eng.named_grads()
    for name, gw in want.items():
        gg = got[name]
        assert _rel(gg, gw) < tol, (name, _rel(gg, gw))


def oracle_output(oracle, x):
    h = x.float()
    with torch.no_grad():
        for layer in oracle.layers.layers:
            h, _, _ = layer.forward_slice(h, None, None)
    return h


def test_engine_graph_step_runs_and_updates():
    from terapipe_b200.models import TransformerConfig
    from terapipe_b200.runtime.engine import StageEngine
    cfg = TransformerConfig(batch_size=2, seq_len=128, n_layers=2, embedding_dim=256,
                            num_attention_heads=4, n_devices=1)
    eng = StageEngine(cfg, [2], [32] * 4, lr=1e-3, init="device", use_graph=True)
    x = torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim).cuda()
    eng.set_input(x)
    before = eng.master.clone()
    losses = []
    for _ in range(4):
        eng.step()
        losses.append(eng.loss().item())
    eng.check_status()
    assert eng._graph is not None
    assert (eng.master - before).abs().max().item() > 0
    assert eng.grad.abs().max().item() == 0.0       # Adam zeroes the accumulator
    assert abs(eng.adam_state[0].item() - 4.0) < 1e-6
    assert all(abs(v) < 10 for v in losses)
    # loss = mean(output) with lr 1e-3 on that very objective must go down
    assert losses[-1] < losses[0]


def test_trainer_step_and_checkpoint_roundtrip(tmp_path):
    from terapipe_b200.runtime import checkpointing as ck
    from terapipe_b200.runtime.trainer import Trainer
    from terapipe_b200.utils.trace import SliceTimeline
    tr = Trainer("test", batch_size=2, n_layers=2, batch_slices=[2], seq_slices=[64, 64], lr=1e-3,
                 use_graph=False)
    tr.engine.timeline = SliceTimeline(stage=0)
    x = tr.synthetic_input(0, pinned=True)
    assert x.is_pinned() and x.shape == (128, 2, 256)
    l0 = tr.train_step(x)
    l1 = tr.train_step(x)
    assert l1 < l0                                   # lr 1e-3 on loss = mean(output)
    recs = tr.engine.timeline.records()
    assert [r["pass"] for r in recs] == ["forward", "forward", "backward", "backward"]
    assert all(r["t_end_ms"] > r["t_start_ms"] for r in recs)
    ck.save_checkpoint(tr.engine, str(tmp_path))
    fresh = Trainer("test", batch_size=2, n_layers=2, batch_slices=[2], seq_slices=[64, 64], lr=1e-3,
                    use_graph=False, seed=5)
    assert not torch.equal(fresh.engine.master, tr.engine.master)
    meta = ck.load_checkpoint(fresh.engine, str(tmp_path))
    assert meta["step"] == 2
    for name in ("master", "exp_avg", "exp_avg_sq", "model", "adam_state"):
        assert torch.equal(getattr(fresh.engine, name), getattr(tr.engine, name)), name
    # both continue identically
    a, b = tr.train_step(x), fresh.train_step(x)
    assert a == b


@pytest.mark.parametrize("heads,hidden", [(4, 320), (4, 384)])
def test_engine_with_head_dim_80_and_96_matches_portable_oracle(heads, hidden, tmp_path):
    """Heads of 80 (gpt3-2b) and 96 columns (megatron-*, gpt3-7hm) run on the 128-wide attention
    kernels with zero-padded projections: outputs, gradients (in the model's own shapes), an
    optimizer step and a checkpoint must match what the unpadded model gives, and the padding
    must stay exactly zero."""
    from terapipe_b200.models import TransformerConfig
    from terapipe_b200.runtime import checkpointing as ck
    from terapipe_b200.runtime.engine import StageEngine
    cfg = TransformerConfig(batch_size=2, seq_len=128, n_layers=2, embedding_dim=hidden,
                            num_attention_heads=heads, n_devices=1)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g).cuda()
    oracle = _oracle(cfg, x)
    eng = StageEngine(cfg, [1, 1], [40, 24, 64], init="reference", use_graph=False, lr=1e-3)
    assert eng.Dk == 128 and eng.D == hidden // heads
    sd = eng.state_dict()
    for (name, a), b in zip(sd.items(), oracle.layers.state_dict().values()):
        assert a.shape == b.shape and _rel(a, b) < 5e-3, name
    eng.set_input(x)
    eng.compute_grads()
    eng.check_status()
    assert abs(eng.loss().item() - oracle.last_loss) < 2e-3
    assert _rel(eng.output(), oracle_output(oracle, x)) < 2e-2
    got = eng.named_grads()
    for name, gw in oracle.named_grads().items():
        assert got[name].shape == gw.shape and _rel(got[name], gw) < 2e-2, (name, _rel(got[name], gw))
    # the padding receives no gradient and an optimizer step leaves it at zero
    eng.grad.zero_()
    for _ in range(2):
        eng.step()
    torch.cuda.synchronize()
    eng.check_status()
    for name in eng._HEAD_PADDED:
        for buf in (eng.master, eng.model, eng.exp_avg_sq):
            w = eng.param(0, name, buf)
            assert w.shape != eng.get_param(0, name, buf).shape
            # dropping the padding and putting zeros back reproduces the buffer
            assert torch.equal(eng._pad_heads(name, eng._unpad_heads(name, w)), w), name
    # a checkpoint holds the model's own shapes and restores the padded buffers
    ck.save_checkpoint(eng, str(tmp_path))
    fresh = StageEngine(cfg, [1, 1], [40, 24, 64], init="device", use_graph=False, lr=1e-3, seed=3)
    ck.load_checkpoint(fresh, str(tmp_path))
    for name in ("master", "exp_avg", "exp_avg_sq", "model"):
        assert torch.equal(getattr(fresh, name), getattr(eng, name)), name
