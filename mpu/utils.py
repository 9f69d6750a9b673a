from terapipe_b200.parallel.utils import *  # noqa: F401,F403
