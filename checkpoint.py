"""Activation recompute usable with ``torch.autograd.grad``:
``CheckpointFunction.apply(run_function, n_tensor_args, *args)``.
Implemented in :mod:`terapipe_b200.utils.checkpoint`."""
from terapipe_b200.utils.checkpoint import (CheckpointFunction, check_backward_validity,  # noqa: F401
                                            detach_variable)
