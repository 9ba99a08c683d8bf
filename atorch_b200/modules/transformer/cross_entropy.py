"""``AtorchCrossEntropyLoss`` (reference: atorch/modules/transformer/cross_entropy.py:7-71): cross-entropy
with ignore_index, label smoothing, z-loss (``lse_square_scale``), in-place backward and an optional
process group over which the vocabulary dimension is split."""
import torch
import torch.nn as nn

from ... import ops


class AtorchCrossEntropyLoss(nn.Module):
    def __init__(self, ignore_index: int = -100, reduction: str = "mean", label_smoothing: float = 0.0,
                 lse_square_scale: float = 0.0, inplace_backward: bool = False, process_group=None):
        super().__init__()
        if reduction not in ("mean", "none", "sum"):
            raise NotImplementedError("reduction must be mean, none or sum")
        self.ignore_index, self.reduction = ignore_index, reduction
        self.label_smoothing, self.lse_square_scale = label_smoothing, lse_square_scale
        self.inplace_backward, self.process_group = inplace_backward, process_group

    def forward(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        shape = target.shape
        loss = ops.cross_entropy(input.reshape(-1, input.shape[-1]), target.reshape(-1), self.ignore_index,
                                 self.label_smoothing, self.lse_square_scale, self.inplace_backward,
                                 self.process_group)
        if self.reduction == "mean":
            return loss.sum() / (target != self.ignore_index).sum().clamp(min=1)
        if self.reduction == "sum":
            return loss.sum()
        return loss.view(shape)


CrossEntropyLoss = AtorchCrossEntropyLoss
