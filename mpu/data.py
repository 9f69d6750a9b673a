from terapipe_b200.parallel.data import *  # noqa: F401,F403
