"""Host helpers (watchdog timeout, seeding, slice arithmetic, memory report).
Implemented in :mod:`terapipe_b200.utils.misc`."""
from terapipe_b200.utils.misc import (TimeoutError, mem_report, set_random_seed,  # noqa: F401
                                      suppress_output, timeout, uniform_slice)
