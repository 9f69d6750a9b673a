"""The command-line drivers and launch scripts on CPU ranks (gloo), tiny model."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _env():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    return env


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


def test_sweep_driver_single_rank_writes_results(tmp_path):
    cmd = [sys.executable, os.path.join(ROOT, "test_transformer_terapipe.py"), "127.0.0.1", "-p",
           _free_port(), "--model", "test", "--n-layers", "2", "--batch-size", "2",
           "--n-batch-slices", "1,2", "--n-input-slices", "4", "--n-steps", "2"]
    subprocess.run(cmd, cwd=tmp_path, env=_env(), check=True, timeout=300)
    results = json.load(open(tmp_path / "results.json"))
    assert len(results) == 2
    for r in results:
        assert r["model"] == "test" and r["n_input_slices"] == 4 and r["mean_time"] > 0
        assert {"n_gpus", "batch_size", "n_batch_slices", "n_steps", "mixed_precision",
                "model_parallel_size", "pipeline_parallel_size", "rank", "data_parallel_size",
                "std_time", "tokens_per_s", "max_over_ranks_device_ms", "peak_memory_gb"} <= set(r)
    lines = [json.loads(l) for l in open(tmp_path / "results.rank0.jsonl")]
    assert lines == results


def test_launch_script_two_stage_pipeline_verify(tmp_path):
    """mpirun_terapipe.sh with PP=2 on two CPU ranks: --verify asserts sliced == unsliced."""
    env = dict(_env(), PORT=_free_port(), PYTHON=sys.executable, TERAPIPE_TIME_LIMIT="240")
    cmd = ["bash", os.path.join(ROOT, "mpirun_terapipe.sh"), "1", "2", "1", "2", "test", "2", "1", "4",
           "1", "--verify", "--n-layers", "2"]
    out = subprocess.run(cmd, cwd=tmp_path, env=env, timeout=400, capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]


def test_module_driver_verify_save_then_load(tmp_path):
    env = dict(_env(), PYTHON=sys.executable, TERAPIPE_TIME_LIMIT="240")
    vdir = str(tmp_path / "v")
    save = ["bash", os.path.join(ROOT, "mpirun_terapipe_new.sh"), "1", "1", "1", "1", "test", "2", "1",
            "1", "1", "--verify", "save", "--verify-path", vdir, "--n-layers", "2"]
    out = subprocess.run(save, cwd=tmp_path, env=dict(env, PORT=_free_port()), timeout=400,
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert sorted(f for f in os.listdir(vdir) if not f.endswith(".lock")) == \
        ["input.pt", "model.ckpt", "model.grad.ckpt"]
    load = ["bash", os.path.join(ROOT, "mpirun_terapipe_new.sh"), "1", "2", "2", "1", "test", "2", "2",
            "4", "1", "--verify", "load", "--verify-path", vdir, "--n-layers", "2"]
    out = subprocess.run(load, cwd=tmp_path, env=dict(env, PORT=_free_port()), timeout=400,
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert out.stdout.count("'ok': True") == 2


def test_planner_scripts_run(tmp_path):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "flop_model.py")], env=_env(),
                         capture_output=True, text=True, timeout=120, check=True)
    assert "9.73" in out.stdout and "gpt3-13b" in out.stdout
    out = subprocess.run([sys.executable, os.path.join(ROOT, "memory_model.py")], env=_env(),
                         capture_output=True, text=True, timeout=120, check=True)
    assert out.stdout.startswith("11.48")


def test_driver_modules_keep_the_reference_public_names():
    """Scripts that import helpers from the drivers keep working after a switch."""
    import importlib
    sys.path.insert(0, ROOT)
    wanted = {
        "terapipe": ["LOSS_SCALE_FACTOR", "loss_func", "initialize_distributed_env", "TransformerLayers",
                     "PipelineSendOperator", "PipelineRecvOperator", "pipeline_send", "pipeline_recv",
                     "TeraPipeBackwardPassHook", "terapipe_backward_hook", "TeraPipe", "initialize_model",
                     "measure_iteration_time", "slice_state_dict", "verify_one_step", "main"],
        "test_transformer_terapipe": ["NCCLTransformer", "NCCLTransformerRunner", "parse_comma_delimited_arg",
                                      "main", "LOSS_SCALE_FACTOR"],
        "terapipe_latency_model": ["TerapipeLatencyModel", "parse_json", "format_json", "main"],
        "p2p_comm_latency": ["p2p_communication_latency", "benchmark_p2p_communication",
                             "get_local_ip_address"],
        "latency_model": ["SCAN_GRID", "STEP_GAP", "SingleLayerLatency", "fit_single_layer_model", "planning",
                          "evaluate_split", "analysis_model", "parse_json", "inputs"],
        "batch_test": ["parse_comma_delimited_arg", "run_experiment", "main"],
        "transformer_models": ["NEG_INF", "MODEL_CONFIGS", "BATCH_CONFIGS", "TransformerConfig", "assign_cache_",
                               "MultiheadLMAttentionWithCache", "TransformerLayer",
                               "ModelParallelMultiheadLMAttentionWithCache", "ModelParallelTransformerLayer",
                               "SingleDeviceTransformer", "grid_slice_batch_and_sequence"],
        "checkpoint": ["CheckpointFunction", "detach_variable", "check_backward_validity"],
        "utils": ["TimeoutError", "timeout", "suppress_output", "set_random_seed", "mem_report", "uniform_slice"],
    }
    for mod, names in wanted.items():
        m = importlib.import_module(mod)
        missing = [n for n in names if not hasattr(m, n)]
        assert not missing, (mod, missing)
