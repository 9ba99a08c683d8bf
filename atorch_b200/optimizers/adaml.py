"""``AdamL``: Adam with an L1 or L2,1 (group-lasso over rows) proximal step after the update, for
sparse embedding tables. ``l1``/``l21`` are the regularisation strengths; the proximal operators are
soft-thresholding of entries / of row norms. (Reference: atorch/optimizers/adaml.py:7.)"""
from __future__ import annotations

import torch
from torch.optim import Adam


class AdamL(Adam):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, amsgrad=False, l1: float = 0.0,
                 l21: float = 0.0):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)
        for g in self.param_groups:
            g.setdefault("l1", l1)
            g.setdefault("l21", l21)

    @torch.no_grad()
    def step(self, closure=None):
        loss = super().step(closure)
        for g in self.param_groups:
            lr, l1, l21 = g["lr"], g.get("l1", 0.0), g.get("l21", 0.0)
            for p in g["params"]:
                if p.grad is None:
                    continue
                if l1 > 0:
                    p.copy_(torch.sign(p) * torch.clamp(p.abs() - lr * l1, min=0.0))
                if l21 > 0 and p.dim() >= 2:
                    rn = torch.linalg.vector_norm(p.reshape(p.shape[0], -1), dim=1).clamp(min=1e-12)
                    shrink = torch.clamp(1.0 - lr * l21 / rn, min=0.0)
                    p.mul_(shrink.view(-1, *([1] * (p.dim() - 1))))
        return loss
