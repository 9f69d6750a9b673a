from terapipe_b200.parallel.cross_entropy import *  # noqa: F401,F403
