"""The checked kernel build (TERAPIPE_CHECKED=1): the same kernels with index checks that report
through the status word.  The library is chosen when it is first loaded, so every case runs in a
child process of its own."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(body: str, checked: bool = True) -> str:
    env = dict(os.environ, TERAPIPE_CHECKED="1" if checked else "0", PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-c", textwrap.dedent(body)], env=env, cwd=ROOT,
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res.stdout


def test_selftest_check_fires_in_the_checked_build_only():
    """A failing check leaves its code in the status word, the host raises CheckFailed, and the
    context stays usable; the regular build compiles the check out."""
    body = """
        import torch
        from terapipe_b200.ops import functional as F
        from terapipe_b200.ops.lib import CheckFailed, check, cuda_lib
        lib = cuda_lib()
        word = F.status_word(torch.device("cuda"))
        word.zero_()
        s = torch.cuda.current_stream().cuda_stream
        check(lib.tp_checked_selftest(3, 8, word.data_ptr(), s), "selftest")      # 0 <= 3 < 8 holds
        torch.cuda.synchronize()
        assert int(word.item()) == 0
        check(lib.tp_checked_selftest(9, 8, word.data_ptr(), s), "selftest")      # 9 < 8 fails
        torch.cuda.synchronize()
        code = int(word.item())
        if lib.tp_checked_build():
            assert code == 129, code
            try:
                F.check_device_status()
            except CheckFailed:
                pass
            else:
                raise AssertionError("CheckFailed was not raised")
        else:
            assert code == 0, code
        a = torch.randn(256, 128, device="cuda").half()
        b = torch.randn(256, 128, device="cuda").half()
        out = torch.empty(256, 256, device="cuda", dtype=torch.float16)
        F.gemm(a, b, out)
        torch.cuda.synchronize()
        F.check_device_status()
        rel = (out.float() - a.float() @ b.float().t()).norm() / (a.float() @ b.float().t()).norm()
        assert rel < 2e-3, rel
        print("build", lib.tp_checked_build())
    """
    assert "build 1" in _run(body, checked=True)
    assert "build 0" in _run(body, checked=False)


def test_engine_steps_are_identical_and_clean_under_the_checked_build():
    """Training steps (GEMM, attention, LayerNorm, Adam; sliced, two batch slices) under the
    checked library: no check fires and the parameters equal those of the regular library bit
    for bit."""
    body = """
        import torch
        from terapipe_b200.models import TransformerConfig
        from terapipe_b200.runtime.engine import StageEngine
        cfg = TransformerConfig(batch_size=2, seq_len=256, n_layers=2, embedding_dim=256,
                                num_attention_heads=4, n_devices=1)
        g = torch.Generator().manual_seed(5)
        eng = StageEngine(cfg, [1, 1], [96, 32, 128], init="device", use_graph=False, lr=1e-3)
        for _ in range(3):
            eng.set_input(torch.randn(cfg.seq_len, cfg.batch_size, cfg.embedding_dim, generator=g))
            eng.step()
        torch.cuda.synchronize()
        eng.check_status()
        print("sum", eng.master.double().sum().item().hex(), eng.exp_avg_sq.double().sum().item().hex())
    """
    a = [ln for ln in _run(body, checked=True).splitlines() if ln.startswith("sum")]
    b = [ln for ln in _run(body, checked=False).splitlines() if ln.startswith("sum")]
    assert a and a == b
