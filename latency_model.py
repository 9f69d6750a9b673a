"""Latency fit + slice-schedule dynamic program; run as a script to write ``dp_results.json``
from the tables in ``performance_model_data/``.
Implemented in :mod:`terapipe_b200.planner.latency_model`."""
from terapipe_b200.planner.latency_model import *  # noqa: F401,F403
from terapipe_b200.planner.latency_model import (SCAN_GRID, STEP_GAP, SingleLayerLatency,  # noqa: F401
                                                 analysis_model, cli, evaluate_split,
                                                 fit_single_layer_model, main, parse_json, planning)

from terapipe_b200.planner.latency_model import B200_SETTINGS as inputs  # noqa: E402,F401  settings list

if __name__ == "__main__":
    cli()
