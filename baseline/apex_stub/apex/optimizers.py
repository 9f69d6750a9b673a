import torch


class FusedAdam(torch.optim.Adam):
    """``torch.optim.Adam`` with the fused multi-tensor CUDA implementation; ``zero_grad()``
    sets gradients to None, as apex's optimizer does."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, **_):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         fused=True)

    def zero_grad(self, set_to_none: bool = True):
        super().zero_grad(set_to_none=True)
