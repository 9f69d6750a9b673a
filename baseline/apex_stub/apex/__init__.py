"""Stand-in for NVIDIA apex, which is not installed on this image and cannot be fetched.

The reference imports ``from apex import optimizers`` and uses only
``optimizers.FusedAdam(params, lr=...)`` (test_transformer_terapipe.py:10,95).  The closest
stock equivalent of apex's multi-tensor Adam is ``torch.optim.Adam(..., fused=True)``.
"""
from . import optimizers  # noqa: F401
