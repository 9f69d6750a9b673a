"""bench.py without a GPU: the block table, the slice schedules and the shared config keys."""
import importlib.util
import inspect
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_module"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_blocks_name_valid_models_layouts_and_slices():
    from terapipe_b200.models import MODEL_CONFIGS
    bench = _bench()
    blocks = dict(bench.HEADLINE_BLOCKS, tp_block=dict(bench.TP_BLOCK, tp=2))
    assert {"headline", "headline_44b", "headline_tp8"} <= set(bench.HEADLINE_BLOCKS)
    for name, spec in blocks.items():
        n_layers, hidden, seq_len, heads = MODEL_CONFIGS[spec["model"]]
        n_layers = spec.get("n_layers") or n_layers
        assert heads % spec["tp"] == 0 and n_layers % spec["pp"] == 0, name
        if name != "tp_block":
            assert spec["tp"] * spec["pp"] == 8, name
        bs, ss = bench.slices_for(spec, seq_len)
        assert sum(bs) == spec["batch"] and sum(ss) == seq_len, name
        # the sequence-parallel mode shards every slice in blocks of 32 rows per rank
        assert all((b * t) % (32 * spec["tp"]) == 0 for b in bs for t in ss), name


def test_headline_matches_the_named_configs():
    bench = _bench()
    h = bench.HEADLINE_BLOCKS
    assert (h["headline"]["model"], h["headline"]["tp"], h["headline"]["pp"], h["headline"]["batch"]) == \
        ("gpt3-13b", 2, 4, 8)
    assert (h["headline_44b"]["model"], h["headline_44b"]["tp"], h["headline_44b"]["pp"],
            h["headline_44b"]["batch"]) == ("gpt3-44b", 4, 2, 4)
    assert (h["headline_tp8"]["model"], h["headline_tp8"]["n_layers"], h["headline_tp8"]["tp"],
            h["headline_tp8"]["batch"], h["headline_tp8"]["seq_slices"]) == ("gpt3-175b", 8, 8, 2, 8)


def test_both_arms_fill_the_same_config_keys():
    bench = _bench()
    keys = set(bench.config_dict())
    sys.path.insert(0, ROOT)
    from baseline import reference_arm
    src_ref = inspect.getsource(reference_arm.ReferenceArm.measure)
    src_ours = inspect.getsource(bench.OursArm.measure)
    for k in keys:
        assert f"{k}=" in src_ref, f"reference arm does not fill config key {k}"
        assert f"{k}=" in src_ours, f"our arm does not fill config key {k}"


def test_block_child_results_survive_a_late_failure_or_time_limit():
    """A block's child prints a JSON line after every complete part; the parent keeps the last
    one when the child later exits with an error or is ended by the time limit."""
    bench = _bench()
    env = dict(os.environ)
    py = sys.executable
    ok = bench.run_block_child([py, "-c", "print('noise'); print('{\"ms_per_step\": 2.0}'); "
                                "print('{\"ms_per_step\": 1.0}')"], env, 30, 30)
    assert ok == {"ms_per_step": 1.0}
    late = bench.run_block_child([py, "-c", "import sys; print('{\"ms_per_step\": 2.0}', flush=True); "
                                  "sys.stderr.write('boom\\n'); sys.exit(3)"], env, 30, 30)
    assert late["ms_per_step"] == 2.0 and late["child_exit_status"] == 3 and late["stderr_tail"] == ["boom"]
    none = bench.run_block_child([py, "-c", "import sys; sys.exit(2)"], env, 30, 30)
    assert "error" in none and "ms_per_step" not in none
    slow = bench.run_block_child([py, "-c", "import time; print('{\"ms_per_step\": 5.0}', flush=True); "
                                  "time.sleep(60)"], env, 3, 3)
    assert slow["timed_out"] is True and slow["ms_per_step"] == 5.0 and slow["limit_s"] == 3
    hung = bench.run_block_child([py, "-c", "import time; time.sleep(60)"], env, 2, 2)
    assert hung["timed_out"] is True and "ms_per_step" not in hung


_FAKE_CHILD = """
import json, os, sys, types
sys.argv = ["bench.py", "--child-block", "headline", "--gpus", "1"]
sys.path.insert(0, {root!r})
import importlib.util
spec = importlib.util.spec_from_file_location("bench_module", os.path.join({root!r}, "bench.py"))
bench = importlib.util.module_from_spec(spec); spec.loader.exec_module(bench)

class Arm:
    name = "ours"
    def setup(self, rank, world, local): return None
    def finish(self): pass
    def measure(self, spec, steps, warmup, tp_comm=None, **kw):
        if tp_comm == {fail!r}:
            raise RuntimeError("peer wait timed out")
        ms = {{"fused": 3.0, "sp": 2.0}}[tp_comm]
        return {{"ms_per_step": ms, "value": 1000.0 / ms, "e2e": None, "config": {{"tp_comm": tp_comm}}}}

bench.make_arm = lambda args: Arm()
bench.child_main(bench.parse_args())
"""


def test_child_block_reports_the_modes_that_completed():
    """A tensor-parallel block measures two communication modes in one child: both complete ->
    the faster one is reported with both listed; the second fails -> the first is still there,
    the failure is listed, and the child ends with a non-zero status."""
    bench = _bench()
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    both = bench.run_block_child([sys.executable, "-c", _FAKE_CHILD.format(root=ROOT, fail="none")], env, 60, 60)
    assert both["ms_per_step"] == 2.0 and both["config"]["tp_comm"] == "sp"
    assert set(both["tp_comm_modes"]) == {"fused", "sp"} and "child_exit_status" not in both
    late = bench.run_block_child([sys.executable, "-c", _FAKE_CHILD.format(root=ROOT, fail="sp")], env, 60, 60)
    assert late["ms_per_step"] == 3.0 and late["child_exit_status"] == 3
    assert "RuntimeError" in late["tp_comm_modes"]["sp"]["error"]
    first = bench.run_block_child([sys.executable, "-c", _FAKE_CHILD.format(root=ROOT, fail="fused")], env, 60, 60)
    assert "error" in first and "ms_per_step" not in first
