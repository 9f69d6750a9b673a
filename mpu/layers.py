from terapipe_b200.parallel.layers import *  # noqa: F401,F403
