"""Strategy-aware gradient-norm clipping.

``clip_grad_norm(model, max_norm, norm_type=2, optimizer=None)`` computes the global norm of all
gradients of the job - across the shard group of a sharded engine, across the tensor-parallel group
for parameters that are split over it (replicated parameters counted once), and over pipeline stages
when a ``pipe`` group exists - then scales the gradients in place. fp16 loss-scaled gradients are
unscaled first through the optimizer's ``unscale_``.
(Reference: atorch/auto/clip_grad_norm.py:17-188.)
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..distributed import distributed as D


def _is_tp_sharded(p) -> bool:
    return bool(getattr(p, "tensor_model_parallel", False) or getattr(p, "_atb_tp_sharded", False))


def clip_grad_norm(model, max_norm: float, norm_type: float = 2.0, optimizer=None) -> torch.Tensor:
    from ..parallel.fsdp import FSDP

    if optimizer is not None and hasattr(optimizer, "unscale_"):
        optimizer.unscale_()
    inner = model
    while not isinstance(inner, FSDP) and hasattr(inner, "module") and isinstance(inner.module, torch.nn.Module):
        inner = inner.module
    if isinstance(inner, FSDP):
        return inner.clip_grad_norm_(max_norm, norm_type)
    params = [p for p in model.parameters() if p.grad is not None]
    if not params:
        return torch.zeros(())
    dev = params[0].device
    tp_group, tp_rank = D.parallel_group("tensor"), D.parallel_rank("tensor") or 0
    pp_group = D.parallel_group("pipe")
    if norm_type == math.inf:
        total = torch.stack([p.grad.detach().abs().max() for p in params]).max().to(dev)
        for g in (tp_group, pp_group):
            if g is not None and dist.get_world_size(g) > 1:
                dist.all_reduce(total, op=dist.ReduceOp.MAX, group=g)
    else:
        acc = torch.zeros((), device=dev, dtype=torch.float32)
        for p in params:
            if tp_group is not None and not _is_tp_sharded(p) and tp_rank != 0:
                continue            # replicated over the tensor group: count once
            acc += torch.linalg.vector_norm(p.grad.detach().float(), norm_type) ** norm_type
        for g in (tp_group, pp_group):
            if g is not None and dist.get_world_size(g) > 1:
                dist.all_reduce(acc, group=g)
        total = acc ** (1.0 / norm_type)
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for p in params:
        p.grad.detach().mul_(coef.to(p.grad.dtype))
    return total
