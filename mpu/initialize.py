from terapipe_b200.parallel.initialize import *  # noqa: F401,F403
