"""``AtorchLayerNorm`` (reference: atorch/modules/normalization/layernorm.py:7) and the fused-LayerNorm alias."""
import torch
import torch.nn as nn

from ... import ops


class AtorchLayerNorm(nn.LayerNorm):
    """Drop-in ``nn.LayerNorm`` whose forward/backward run on the sm_100a row kernels."""

    @classmethod
    def from_module(cls, src: nn.LayerNorm, **kwargs):
        m = cls(src.normalized_shape, eps=src.eps, elementwise_affine=src.elementwise_affine,
                bias=src.bias is not None, device=src.weight.device if src.weight is not None else None,
                dtype=src.weight.dtype if src.weight is not None else None)
        if src.weight is not None:
            m.weight = src.weight
        if src.bias is not None:
            m.bias = src.bias
        return m

    def forward(self, x):
        if self.weight is None or len(self.normalized_shape) != 1:
            return super().forward(x)
        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)
        b = None if self.bias is None else (self.bias if self.bias.dtype == x.dtype else self.bias.to(x.dtype))
        return ops.layer_norm(x, w, b, self.eps)


LayerNorm = AtorchLayerNorm
FusedLayerNorm = AtorchLayerNorm
