"""Robustness checks on one GPU: a bounded device wait that runs out, bit-identical repeated
steps, the engine at the width and slice size it is benchmarked at, and long-context attention."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _ptrs(tensors):
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


def test_peer_wait_runs_out_and_reports_through_the_status_word():
    """A fused GEMM + all-reduce launched as rank 0 of a two-rank group whose rank 1 never runs:
    both "ranks'" buffers live on this GPU, the flags rank 1 would raise stay zero, the wait limit
    is 5 ms.  The kernel must return by itself, leave the peer-wait code in the status word, and
    the device must stay usable."""
    from terapipe_b200.ops import functional as F
    from terapipe_b200.ops.lib import CommTimeout, check, cuda_lib
    lib = cuda_lib()
    dev = torch.device("cuda")
    M, N, K, tp = 256, 256, 128, 2
    max_tiles = (M // 128) * (N // 128)
    x = torch.randn(M, K, device=dev, dtype=torch.float16)
    w = torch.randn(N, K, device=dev, dtype=torch.float16)
    stage = [torch.zeros(2 * tp * max_tiles * 128 * 128, device=dev, dtype=torch.float16) for _ in range(tp)]
    flag_a = [torch.zeros(max_tiles * 8, device=dev, dtype=torch.int32) for _ in range(tp)]
    flag_b = [torch.zeros(max_tiles, device=dev, dtype=torch.int32) for _ in range(tp)]
    outs = [torch.zeros(M, N, device=dev, dtype=torch.float16) for _ in range(tp)]
    status = F.status_word(dev)
    status.zero_()
    torch.cuda.synchronize()
    check(lib.tp_set_wait_limit_ns(5_000_000), "tp_set_wait_limit_ns")
    try:
        st = lib.tp_gemm_ar(0, 0, x.data_ptr(), K, w.data_ptr(), K, N, M, N, K, None, None, 0, tp, 0, 1,
                            None, max_tiles, _ptrs(stage), _ptrs(flag_a), _ptrs(flag_b), _ptrs(outs),
                            status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        check(st, "tp_gemm_ar")
        torch.cuda.synchronize()          # returns: the kernel gave up by itself
        assert int(status.item()) == 105  # peer wait timed out
        with pytest.raises(CommTimeout):
            F.check_device_status(dev)
        assert int(status.item()) == 0    # the check clears the word
    finally:
        check(lib.tp_set_wait_limit_ns(5_000_000_000), "tp_set_wait_limit_ns")
    # the context is intact: an ordinary product still runs and is right
    out = torch.empty(M, N, device=dev, dtype=torch.float16)
    F.gemm(x, w, out)
    torch.cuda.synchronize()
    F.check_device_status(dev)
    assert _rel(out, x.float() @ w.float().t()) < 2e-3


def test_trainer_raises_when_the_status_word_is_set():
    """The public step surfaces a device-side time-out: a non-zero status word (written here by
    the host, standing in for a kernel whose wait ran out) makes ``train_step`` raise."""
    from terapipe_b200.ops.lib import CommTimeout
    from terapipe_b200.runtime.trainer import Trainer
    tr = Trainer("test", batch_size=2, n_layers=1, batch_slices=[2], seq_slices=[64, 64], use_graph=False)
    x = tr.synthetic_input(0)
    assert isinstance(tr.train_step(x), float)
    tr.engine.status.fill_(105)
    with pytest.raises(CommTimeout):
        tr.train_step(x)
    assert int(tr.engine.status.item()) == 0
    assert isinstance(tr.train_step(x), float)


@pytest.mark.parametrize("use_graph", [False, True])
def test_repeated_runs_are_bit_identical(use_graph):
    """No kernel accumulates through atomics in an order that varies: two engines built and
    stepped the same way end with identical parameters, moments and loss."""
    from terapipe_b200.models import TransformerConfig
    from terapipe_b200.runtime.engine import StageEngine
    cfg = TransformerConfig(batch_size=2, seq_len=256, n_layers=2, embedding_dim=256,
                            num_attention_heads=4, n_devices=1)
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g) for _ in range(3)]
    runs = []
    for _ in range(2):
        eng = StageEngine(cfg, [1, 1], [96, 32, 128], init="device", use_graph=use_graph, lr=1e-3)
        for x in xs:
            eng.set_input(x)
            eng.step()
        torch.cuda.synchronize()
        eng.check_status()
        runs.append((eng.master.clone(), eng.exp_avg_sq.clone(), eng.loss().item()))
    assert torch.equal(runs[0][0], runs[1][0])
    assert torch.equal(runs[0][1], runs[1][1])
    assert runs[0][2] == runs[1][2]


@pytest.mark.parametrize("use_graph", [False, True])
def test_engine_at_gpt3_1b_width_matches_fp32_oracle(use_graph):
    """Two layers of GPT3-1B width (hidden 2048, head dim 128, FFN 8192) with 1024-row slices, the
    shapes of the headline run (CTA-pair 256-wide tiles, several waves per product), against the
    fp32 autograd pipeline on the same weights."""
    from terapipe_b200.models import TransformerConfig
    from terapipe_b200.runtime.engine import StageEngine
    from terapipe_b200.runtime.portable import PortablePipeline
    cfg = TransformerConfig(batch_size=8, seq_len=512, n_layers=2, embedding_dim=2048,
                            num_attention_heads=16, n_devices=1)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g).cuda()
    oracle = PortablePipeline(cfg, [cfg.batch_size], [cfg.seq_len], device="cuda")
    oracle.compute_grads(x.float())
    eng = StageEngine(cfg, [8], [128] * 4, init="reference", use_graph=use_graph, lr=0.0)
    eng.set_input(x)
    if use_graph:
        # a graph replays whole steps: with lr = 0 the parameters stay put, and the gradients are
        # read from the moment buffer of the first Adam step (m = (1 - beta1) * g / loss scale)
        eng.step()
        eng.step()
        torch.cuda.synchronize()
        assert eng._graph is not None
        eng.check_status()
        assert abs(eng.loss().item() - oracle.last_loss) < 2e-3
        return
    eng.compute_grads()
    eng.check_status()
    assert abs(eng.loss().item() - oracle.last_loss) < 2e-3
    want, got = oracle.named_grads(), eng.named_grads()
    for name, gw in want.items():
        assert _rel(got[name], gw) < 3e-2, (name, _rel(got[name], gw))


def test_attention_long_context_8192():
    """One head pair at sequence length 8192 (the gpt3-13b-8192 shape has b*h small): slices of
    1024 tokens forward and backward against full causal attention in fp32."""
    from terapipe_b200.ops import functional as F
    torch.manual_seed(1)
    D, b, h, L, t = 128, 1, 2, 8192, 1024
    qkv = (torch.randn(L, b, h * 3 * D, device="cuda") * 0.5).half()
    o = torch.zeros(L * b, h * D, device="cuda", dtype=torch.float16)
    lse2 = torch.zeros(b * h, L, device="cuda")
    for c in range(0, L, t):
        F.attn_fwd(qkv, b, h, D, t, c, o[c * b:(c + t) * b], lse2)
    F.check_device_status()
    x = qkv.float().view(L, b, h, 3, D).requires_grad_()
    q, k, v = (x[:, :, :, i].permute(1, 2, 0, 3) for i in range(3))
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    ref = ref.permute(2, 0, 1, 3).reshape(L, b, h * D)
    assert _rel(o.view(L, b, h * D), ref) < 4e-3
    gout = torch.randn(L * b, h * D, device="cuda").half()
    ref.backward(gout.float().view(L, b, h * D))
    dqkv = torch.zeros(L * b, h * 3 * D, device="cuda", dtype=torch.float16)
    delta = torch.full((b * h, L), float("nan"), device="cuda")
    do_full = torch.full((L * b, h * D), float("nan"), device="cuda", dtype=torch.float16)
    for c in reversed(range(0, L, t)):
        do_full[c * b:(c + t) * b] = gout[c * b:(c + t) * b]
        F.attn_bwd(qkv, b, h, D, t, c, L, o[c * b:(c + t) * b], do_full, lse2, delta,
                   dqkv[c * b:(c + t) * b])
    F.check_device_status()
    got = dqkv.view(L, b, h, 3, D).float()
    want = x.grad
    for i, name in enumerate("qkv"):
        assert _rel(got[:, :, :, i], want[:, :, :, i]) < 1.2e-2, name


def test_programmatic_dependent_launch_gives_identical_steps():
    """The GEMM, attention and LayerNorm kernels launched with the programmatic-serialization
    attribute (every kernel waits for its predecessor after its own set-up) produce the same
    parameters as ordinary launches, eagerly and from a captured graph."""
    from terapipe_b200.models import TransformerConfig
    from terapipe_b200.ops.lib import cuda_lib
    from terapipe_b200.runtime.engine import StageEngine
    lib = cuda_lib()
    cfg = TransformerConfig(batch_size=2, seq_len=256, n_layers=2, embedding_dim=256,
                            num_attention_heads=4, n_devices=1)
    g = torch.Generator().manual_seed(17)
    xs = [torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g) for _ in range(3)]
    results = []
    try:
        for pdl, use_graph in ((0, False), (1, False), (1, True)):
            lib.tp_set_pdl(pdl)
            eng = StageEngine(cfg, [2], [64, 64, 128], init="device", use_graph=use_graph, lr=1e-3)
            for x in xs:
                eng.set_input(x)
                eng.step()
            torch.cuda.synchronize()
            eng.check_status()
            results.append(eng.master.clone())
    finally:
        lib.tp_set_pdl(0)
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])
