"""``AtorchRmsNorm``: RMSNorm module on the sm_100a row kernels (reference: atorch/modules/transformer/rmsnorm.py:12)."""
import torch
import torch.nn as nn

from ... import ops


class AtorchRmsNorm(nn.Module):
    def __init__(self, hidden_size, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        if isinstance(hidden_size, (tuple, list, torch.Size)):
            assert len(hidden_size) == 1
            hidden_size = hidden_size[0]
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.variance_epsilon = eps

    def reset_parameters(self):
        nn.init.ones_(self.weight)

    def forward(self, x, residual=None):
        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)
        return ops.rms_norm(x, w, self.variance_epsilon, residual)

    def extra_repr(self):
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"
