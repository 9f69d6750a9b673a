from .misc import (TimeoutError, mem_report, set_random_seed, suppress_output, timeout,
                   uniform_slice)
from . import checkpoint
