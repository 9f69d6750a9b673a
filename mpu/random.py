from terapipe_b200.parallel.random import *  # noqa: F401,F403
