"""Peak-memory models.  Implemented in :mod:`terapipe_b200.planner.memory_model`."""
from terapipe_b200.planner.memory_model import (engine_memory_per_gpu, memory_stats,  # noqa: F401
                                                peak_memory_per_gpu)

if __name__ == "__main__":
    print(peak_memory_per_gpu("gpt3-175b", 1, 32))
    print(peak_memory_per_gpu("gpt3-175b", 1, 48))
    memory_stats("gpt3-175b", 1536)
    memory_stats("gpt3-175b", 2)
