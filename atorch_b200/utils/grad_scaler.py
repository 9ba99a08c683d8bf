"""Gradient scalers.

``DynamicGradScaler`` is a self-contained loss scaler (scale the loss, unscale the gradients, skip the
step and back off when a gradient is not finite, grow after ``growth_interval`` clean steps). The
non-finite flag is one device scalar, reduced with MAX over any number of process groups before the
decision, so that all ranks of a sharded / tensor- / pipeline-parallel job skip together.

``BF16GradScaler`` and ``BF16ShardedGradScaler`` keep the scale at 1: bf16 needs no loss scaling, they only
check for non-finite gradients and skip the step (``amp_native`` with ``skip_if_nonfinite``).
(Reference: atorch/utils/grad_scaler.py:18-88, which derives them from torch's GradScaler /
ShardedGradScaler with frozen scale factors.)
"""
from __future__ import annotations

import sys
from typing import Dict, Iterable, Optional, Sequence

import torch
import torch.distributed as dist


def _grads_of(optimizer) -> Iterable[torch.Tensor]:
    for g in optimizer.param_groups:
        for p in g["params"]:
            if p.grad is not None:
                yield p.grad


class DynamicGradScaler:
    def __init__(self, init_scale: float = 2.0 ** 16, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True,
                 process_groups: Sequence[Optional[dist.ProcessGroup]] = (), min_scale: float = 1.0,
                 max_scale: float = 2.0 ** 24):
        self._scale = float(init_scale)
        self.growth_factor, self.backoff_factor, self.growth_interval = growth_factor, backoff_factor, growth_interval
        self.enabled = enabled
        self.process_groups = list(process_groups)
        self.min_scale, self.max_scale = min_scale, max_scale
        self._good_steps = 0
        self._found_inf: Optional[torch.Tensor] = None      # device scalar of the current step
        self._unscaled: Dict[int, bool] = {}
        self.overflow = False

    # -------------------------------------------------------------------------------------------
    def get_scale(self) -> float:
        return self._scale if self.enabled else 1.0

    def is_enabled(self) -> bool:
        return self.enabled

    def scale(self, outputs):
        if not self.enabled:
            return outputs
        self.overflow = False
        if isinstance(outputs, torch.Tensor):
            return outputs * self._scale
        return type(outputs)(self.scale(o) for o in outputs)

    def unscale_(self, optimizer) -> None:
        """Divide the gradients by the scale and record whether any of them is not finite."""
        if not self.enabled or self._unscaled.get(id(optimizer)):
            return
        inv = 1.0 / self._scale
        flag = None
        for g in _grads_of(optimizer):
            if inv != 1.0:
                g.mul_(inv)
            bad = (~torch.isfinite(g)).any().float() if g.numel() else None
            if bad is not None:
                flag = bad if flag is None else torch.maximum(flag, bad)
        if flag is None:
            flag = torch.zeros(())
        if dist.is_available() and dist.is_initialized():
            for pg in (self.process_groups or []):
                dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=pg)
        self._found_inf = flag if self._found_inf is None else torch.maximum(self._found_inf, flag.to(self._found_inf.device))
        self._unscaled[id(optimizer)] = True

    def step(self, optimizer, *args, **kwargs):
        if not self.enabled:
            return optimizer.step(*args, **kwargs)
        self.unscale_(optimizer)
        if bool(self._found_inf.item()):
            self.overflow = True
            return None
        return optimizer.step(*args, **kwargs)

    def update(self, new_scale: Optional[float] = None) -> None:
        if not self.enabled:
            return
        if new_scale is not None:
            self._scale = float(new_scale)
        elif self._found_inf is not None and bool(self._found_inf.item()):
            self._scale = max(self._scale * self.backoff_factor, self.min_scale)
            self._good_steps = 0
        else:
            self._good_steps += 1
            if self._good_steps >= self.growth_interval:
                self._scale = min(self._scale * self.growth_factor, self.max_scale)
                self._good_steps = 0
        self._found_inf = None
        self._unscaled.clear()

    def has_overflow(self) -> bool:
        return self.overflow

    def state_dict(self) -> dict:
        return {"scale": self._scale, "growth_factor": self.growth_factor, "backoff_factor": self.backoff_factor,
                "growth_interval": self.growth_interval, "_growth_tracker": self._good_steps}

    def load_state_dict(self, sd: dict) -> None:
        self._scale = float(sd["scale"])
        self.growth_factor = sd.get("growth_factor", self.growth_factor)
        self.backoff_factor = sd.get("backoff_factor", self.backoff_factor)
        self.growth_interval = sd.get("growth_interval", self.growth_interval)
        self._good_steps = int(sd.get("_growth_tracker", 0))


class BF16GradScaler(DynamicGradScaler):
    """Scale fixed at 1: only the non-finite check and the skipped step remain."""

    def __init__(self, init_scale=2.0 ** 16, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000, enabled=True,
                 process_groups: Sequence[Optional[dist.ProcessGroup]] = ()):
        super().__init__(1.0, 1.0, 1.0, sys.maxsize, enabled, process_groups)


class BF16ShardedGradScaler(BF16GradScaler):
    """The same for sharded parameters: the flag is reduced over the shard group, since every rank
    only sees its own part of the gradients."""

    def __init__(self, init_scale=2.0 ** 16, backoff_factor=0.5, growth_factor=2.0, growth_interval=2000, enabled=True,
                 process_group=None):
        super().__init__(enabled=enabled, process_groups=[process_group])


class ShardedGradScaler(DynamicGradScaler):
    """Dynamic fp16 loss scaling for sharded parameters (flag reduced over the shard group)."""

    def __init__(self, init_scale=2.0 ** 16, backoff_factor=0.5, growth_factor=2.0, growth_interval=2000, enabled=True,
                 process_group=None):
        super().__init__(init_scale, growth_factor, backoff_factor, growth_interval, enabled, [process_group])
