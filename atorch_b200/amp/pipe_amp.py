"""Loss scaling under pipeline parallelism.

With pipeline parallelism every rank holds some stages and sees only their gradients, but all stages must
take the same decision: skip the step and back off the scale, or step. ``PipeGradScaler`` collects the
non-finite flags of every local stage optimizer, sums them over the ``pipe`` group (one all-reduce of one
scalar per step, issued once even when several local stages call in) and only then steps or skips.
(Reference: atorch/amp/pipe_amp.py:51-288, built on torch's GradScaler with a condition variable across
RPC-driven stage threads; here stages of one rank run in one thread, so a counter is enough.)
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..utils.grad_scaler import DynamicGradScaler


class PipeGradScaler(DynamicGradScaler):
    def __init__(self, init_scale=2.0 ** 16, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000, enabled=True,
                 pipe_group: Optional[dist.ProcessGroup] = None, num_local_stages: int = 1):
        if pipe_group is None and dist.is_available() and dist.is_initialized():
            from ..distributed import distributed as D

            pipe_group = D.parallel_group("pipe") or D.parallel_group("pipeline")
        super().__init__(init_scale, growth_factor, backoff_factor, growth_interval, enabled,
                         [pipe_group] if pipe_group is not None else [])
        self.num_local_stages = num_local_stages
        self._pending: List = []

    def unscale_(self, optimizer) -> None:
        """Unscale one local stage's gradients; the cross-stage reduction waits for the last local stage."""
        if not self.enabled or self._unscaled.get(id(optimizer)):
            return
        groups, self.process_groups = self.process_groups, []       # local check only
        try:
            super().unscale_(optimizer)
        finally:
            self.process_groups = groups
        self._pending.append(optimizer)
        if len(self._pending) >= self.num_local_stages and dist.is_available() and dist.is_initialized():
            for pg in self.process_groups:
                dist.all_reduce(self._found_inf, op=dist.ReduceOp.SUM, group=pg)
            self._found_inf = (self._found_inf > 0).float()

    def step(self, optimizer, *args, **kwargs):
        if not self.enabled:
            return optimizer.step(*args, **kwargs)
        self.unscale_(optimizer)
        if len(self._pending) < self.num_local_stages:
            raise RuntimeError("PipeGradScaler.step: unscale_ every local stage's optimizer before the first step "
                               f"({len(self._pending)} of {self.num_local_stages} seen)")
        if bool(self._found_inf.item()):
            self.overflow = True
            return None
        return optimizer.step(*args, **kwargs)

    def update(self, new_scale=None) -> None:
        super().update(new_scale)
        self._pending.clear()
