"""Host-side auxiliary subsystems: watchdog/heartbeats, launcher reaping, checkpoint re-sharding."""
import os
import sys
import time

import torch

from terapipe_b200.utils import launcher
from terapipe_b200.utils.watchdog import Watchdog, stale_ranks


def test_watchdog_fires_only_without_beats(tmp_path):
    fired = []
    wd = Watchdog(0.3, rank=3, heartbeat_dir=str(tmp_path), on_timeout=lambda: fired.append(1),
                  poll_s=0.05).start()
    for _ in range(6):
        time.sleep(0.1)
        wd.beat()
    assert not fired and stale_ranks(str(tmp_path), 4, 5.0) == [0, 1, 2]
    time.sleep(0.6)
    wd.stop()
    assert fired and wd.fired


def test_launcher_reaps_job_when_a_rank_fails(tmp_path):
    script = tmp_path / "job.py"
    script.write_text(
        "import os, sys, time\n"
        "rank = int(os.environ['RANK'])\n"
        "assert os.environ['OMPI_COMM_WORLD_SIZE'] == os.environ['WORLD_SIZE'] == '3'\n"
        "if rank == 1:\n    sys.exit(7)\n"
        "time.sleep(60)\n")
    t0 = time.time()
    status = launcher.launch([sys.executable, str(script)], nproc=3)
    assert status == 7 and time.time() - t0 < 20


def test_launcher_time_limit(tmp_path):
    script = tmp_path / "sleep.py"
    script.write_text("import time\ntime.sleep(60)\n")
    t0 = time.time()
    assert launcher.launch([sys.executable, str(script)], nproc=2, timeout=1.0) == 124
    assert time.time() - t0 < 20


class _FakeEngine:
    """The attributes of StageEngine that checkpointing touches, on the CPU."""

    def __init__(self, n_layers_total, tp, pp, tp_idx, pp_idx, H=16):
        from terapipe_b200.parallel.topology import Topology
        from terapipe_b200.runtime.engine import _Layout
        self.tp, self.pp, self.dp, self.tp_idx, self.pp_idx, self.dp_idx = tp, pp, 1, tp_idx, pp_idx, 0
        ids = Topology(tp * pp, tp, pp).layers_of_stage(n_layers_total, pp_idx)
        self.n_layers = len(ids)
        self.layout = _Layout(self.n_layers, H, 4 * H, tp)
        n = self.layout.total
        self.master, self.exp_avg, self.exp_avg_sq = (torch.zeros(n) for _ in range(3))
        self.model = torch.zeros(n)
        self.adam_state = torch.zeros(3)
        self.step_count, self.loss_scale = 0, 128.0

        class Cfg:
            n_layers = n_layers_total
        self.cfg = Cfg()

    def param(self, layer, name, buf=None):
        import math
        buf = self.model if buf is None else buf
        shape = self.layout.shapes[name]
        off = self.layout.offsets[layer][name]
        return buf[off:off + math.prod(shape)].view(shape)

    get_param = param

    def set_param(self, layer, name, value, buf=None):
        self.param(layer, name, buf).copy_(value)


def test_checkpoint_roundtrip_and_reshard(tmp_path):
    from terapipe_b200.runtime import checkpointing as ck
    src, dst = str(tmp_path / "a"), str(tmp_path / "b")
    torch.manual_seed(0)
    full = {}
    engines = {}
    for s in range(2):
        for r in range(2):
            e = _FakeEngine(3, 2, 2, r, s)
            engines[(s, r)] = e
    # fill from a full (unsharded) random state so shards are mutually consistent
    from terapipe_b200.models import slice_state_dict
    from terapipe_b200.runtime.engine import PARAM_ORDER, _Layout
    lay = _Layout(3, 16, 64, 1)
    for l in range(3):
        for name in PARAM_ORDER:
            full[f"layers.layers.{l}.{name}"] = torch.randn(lay.shapes[name])
    for (s, r), e in engines.items():
        sd = slice_state_dict(3, full, 2, r, 2, s)
        for l in range(e.n_layers):
            for name in PARAM_ORDER:
                e.param(l, name, e.master).copy_(sd[f"layers.layers.{l}.{name}"])
                e.param(l, name, e.exp_avg).copy_(2 * sd[f"layers.layers.{l}.{name}"])
        e.step_count = 11
        e.adam_state.copy_(torch.tensor([11.0, 0.5, 0.25]))
        ck.save_checkpoint(e, src)
    assert sorted(os.listdir(src)) == [f"shard_pp{s}_tp{r}_dp0.pt" for s in range(2) for r in range(2)]
    # same layout: restore into a fresh engine
    fresh = _FakeEngine(3, 2, 2, 1, 0)
    meta = ck.load_checkpoint(fresh, src)
    assert meta["step"] == 11 and torch.equal(fresh.master, engines[(0, 1)].master)
    assert torch.equal(fresh.exp_avg, engines[(0, 1)].exp_avg) and fresh.adam_state[1] == 0.5
    # other layout: tp 2 x pp 2  ->  tp 1 x pp 3
    ck.reshard(src, dst, tp=1, pp=3)
    for s in range(3):
        e = _FakeEngine(3, 1, 3, 0, s)
        ck.load_checkpoint(e, dst)
        for name in PARAM_ORDER:
            assert torch.equal(e.param(0, name, e.master), full[f"layers.layers.{s}.{name}"]), name
            assert torch.equal(e.param(0, name, e.exp_avg), 2 * full[f"layers.layers.{s}.{name}"])


def test_launch_plan_records_once_and_replays():
    """Recorded launch plans of the engine (host logic only; a fake kernel library)."""
    from terapipe_b200.runtime.launch_plan import RecordingLibrary, SegmentCache

    class FakeLib:
        def __init__(self):
            self.log = []
            self.fail_next = False

        def tp_a(self, x, y):
            self.log.append(("a", x, y))
            return 0

        def tp_b(self, x):
            self.log.append(("b", x))
            rc, self.fail_next = (-3 if self.fail_next else 0), False
            return rc

    fake = FakeLib()
    lib = RecordingLibrary(fake)
    cache = SegmentCache(lib)
    derived = []

    def segment(i):            # argument derivation happens only while recording
        derived.append(i)
        lib.tp_a(i, 10 * i)
        lib.tp_b(i + 1)

    cache.validate("stream0")
    for _ in range(3):
        cache.run(("fwd", 0), segment, 1)
        cache.run(("fwd", 1), segment, 2)
    assert derived == [1, 2]                                   # recorded once per key
    assert fake.log == [("a", 1, 10), ("b", 2), ("a", 2, 20), ("b", 3)] * 3
    assert cache.replayed == 8
    lib.tp_a(7, 7)                                             # calls outside a segment just run
    assert fake.log[-1] == ("a", 7, 7) and len(cache.segments) == 2
    cache.validate("stream1")                                  # new token: recordings dropped
    assert not cache.segments
    fake.fail_next = True
    cache.run(("fwd", 0), segment, 1)                          # a failing launch is not cached
    assert ("fwd", 0) not in cache.segments
    cache.run(("fwd", 0), segment, 1)
    assert ("fwd", 0) in cache.segments
