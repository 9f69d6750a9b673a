"""FLOP model of a training iteration; run as a script to print the efficiency of the published
V100-cluster latencies.  Implemented in :mod:`terapipe_b200.planner.flop_model`."""
from terapipe_b200.planner.flop_model import *  # noqa: F401,F403
from terapipe_b200.planner.flop_model import efficiency_stats, flop_stats, main  # noqa: F401

if __name__ == "__main__":
    main()
