"""Recorded launch plans on the real engine: replayed steps must equal derived ones bit for bit.
(The recorder itself is covered on CPU in tests/test_aux_cpu.py.)"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_replayed_steps_match_derived_steps():
    from terapipe_b200.models import TransformerConfig
    from terapipe_b200.runtime.engine import StageEngine
    cfg = TransformerConfig(batch_size=2, seq_len=128, n_layers=2, embedding_dim=256,
                            num_attention_heads=4, n_devices=1)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g) for _ in range(3)]
    models = []
    for plan in (False, True):
        eng = StageEngine(cfg, [1, 1], [32, 96], init="device", use_graph=False, lr=1e-3,
                          launch_plan=plan)
        assert (eng._plan is not None) == plan
        for x in xs:
            eng.set_input(x)
            eng.step()
        torch.cuda.synchronize()
        eng.check_status()
        if plan:
            assert eng._plan.replayed > 0 and len(eng._plan.segments) == 2 * 2 * 2 + 1
        models.append((eng.model.clone(), eng.loss().item()))
    assert torch.equal(models[0][0], models[1][0])
    assert models[0][1] == models[1][1]


def test_segment_graph_steps_match_eager_steps():
    """Per-segment CUDA graphs (the default for stages that cannot capture the whole step):
    steps replayed from the segment graphs equal eagerly launched steps bit for bit."""
    from terapipe_b200.models import TransformerConfig
    from terapipe_b200.runtime.engine import StageEngine
    cfg = TransformerConfig(batch_size=2, seq_len=128, n_layers=2, embedding_dim=256,
                            num_attention_heads=4, n_devices=1)
    g = torch.Generator().manual_seed(6)
    xs = [torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g) for _ in range(4)]
    models = []
    for seg in (False, True):
        eng = StageEngine(cfg, [1, 1], [32, 96], init="device", use_graph=False, lr=1e-3,
                          launch_plan=False, segment_graphs=seg)
        assert (eng._seg_graphs is not None) == seg
        for x in xs:
            eng.set_input(x)
            eng.step()
        torch.cuda.synchronize()
        eng.check_status()
        if seg:
            # 2 batch slices x 2 token slices x (forward, backward) + weight gradients + update
            assert len(eng._seg_graphs) == 2 * 2 * 2 + 2
            assert all(ent[0] is not None for ent in eng._seg_graphs.values())
        models.append((eng.model.clone(), eng.loss().item()))
    assert torch.equal(models[0][0], models[1][0])
    assert models[0][1] == models[1][1]
