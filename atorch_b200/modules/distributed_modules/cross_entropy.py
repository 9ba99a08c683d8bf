"""Vocabulary-parallel cross entropy: each rank holds ``[tokens, V / tp]`` logits and global label
ids. Runs on the sm_100a split-vocabulary kernel (per-rank lse / label logit, one all-gather and
one all-reduce of per-token scalars) or on its PyTorch evaluation on CPU.
(Reference: atorch/modules/distributed_modules/cross_entropy.py:9-127.)
"""
from __future__ import annotations

import torch

from ... import ops
from ...distributed import distributed as D


def vocab_parallel_cross_entropy(vocab_parallel_logits: torch.Tensor, target: torch.Tensor, group=None,
                                 label_smoothing: float = 0.0, ignore_index: int = -100) -> torch.Tensor:
    """Per-token losses shaped like ``target``."""
    group = group if group is not None else D.parallel_group("tensor")
    shape = target.shape
    loss = ops.cross_entropy(vocab_parallel_logits.reshape(-1, vocab_parallel_logits.shape[-1]),
                             target.reshape(-1), ignore_index=ignore_index, label_smoothing=label_smoothing,
                             process_group=group)
    return loss.view(shape)


class VocabParallelCrossEntropyLoss(torch.nn.Module):
    def __init__(self, group=None, ignore_index: int = -100, reduction: str = "mean"):
        super().__init__()
        self.group, self.ignore_index, self.reduction = group, ignore_index, reduction

    def forward(self, logits, target):
        loss = vocab_parallel_cross_entropy(logits, target, self.group, ignore_index=self.ignore_index)
        if self.reduction == "mean":
            return loss.sum() / (target != self.ignore_index).sum().clamp(min=1)
        if self.reduction == "sum":
            return loss.sum()
        return loss
