from terapipe_b200.parallel.mappings import *  # noqa: F401,F403
