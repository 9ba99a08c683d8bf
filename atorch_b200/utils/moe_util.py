"""Norms and clipping for models whose parameters are partitioned over different process groups (dense parameters
replicated or sharded over the data group, expert parameters distinct per expert-parallel rank), and small file
helpers for expert checkpoints.

A parameter states where its pieces live in one of three ways: it is a ``DTensor`` (its device mesh), it carries
``p.norm_group`` (a process group; ``None`` = whole on every rank), or it is tagged as an expert parameter
(``p.expert`` / ``p.is_expert`` / ``p.allreduce is False``) while an ``"expert"`` parallel group exists. Parameters are
bucketed by that group; each bucket's local ``sum |x|^p`` (or max) is all-reduced over its own group only, then the
buckets are combined. Everything else is counted once, locally.
(Reference: atorch/utils/moe_util.py:27-38, 416-421, 505-590; the safetensors-to-FSDP2 loaders there are tied to
DTensor layouts and have their counterpart in ``utils/safetensors_io.py``.)
"""
from __future__ import annotations

import math
import os
from typing import Dict, Iterable, List, Optional, Union

import torch
import torch.distributed as dist

from ..distributed import distributed as D


def has_file_with_suffix(path: str, suffix: str) -> bool:
    return any(f.endswith(suffix) for f in os.listdir(path))


def get_files_with_suffix(path: str, suffix: str) -> List[str]:
    return [f for f in os.listdir(path) if f.endswith(suffix)]


def move_optimizer_state(optimizer: torch.optim.Optimizer, device="cpu") -> None:
    """Every tensor of the optimizer state to ``device`` (to make room for generation or evaluation, and back)."""
    for state in optimizer.state.values():
        for k, v in state.items():
            if isinstance(v, torch.Tensor):
                state[k] = v.to(device)


def _is_expert(p) -> bool:
    return bool(getattr(p, "expert", False) or getattr(p, "is_expert", False) or getattr(p, "allreduce", True) is False)


def _norm_group(p):
    """(key, process group or None, local tensor getter) of a parameter."""
    if hasattr(p, "norm_group"):
        g = p.norm_group
        return (id(g) if g is not None else None), g
    if _is_expert(p):
        g = D.parallel_group("expert")
        if g is not None and dist.get_world_size(g) > 1:
            return id(g), g
    return None, None


def _local(t):
    return t.to_local() if hasattr(t, "to_local") else t


def compute_norm_(parameters: Union[torch.Tensor, Iterable[torch.Tensor]], norm_type: float = 2.0,
                  error_if_nonfinite: bool = False, foreach: Optional[bool] = None, grad: bool = False) -> torch.Tensor:
    if isinstance(parameters, torch.Tensor):
        parameters = [parameters]
    norm_type = float(norm_type)
    buckets: Dict[object, list] = {}
    for p in parameters:
        t = p.grad if grad else p
        if t is None:
            continue
        if hasattr(t, "device_mesh") and hasattr(t, "full_tensor"):      # DTensor: its own reduction
            n = torch.linalg.vector_norm(t.detach().float(), norm_type)
            n = n.full_tensor() if hasattr(n, "full_tensor") else n
            buckets.setdefault(("dtensor", id(t.device_mesh)), [None, []])[1].append(n ** (1 if math.isinf(norm_type) else norm_type))
            continue
        key, g = _norm_group(p)
        b = buckets.setdefault(key, [g, []])
        x = _local(t).detach().float()
        b[1].append(x.abs().max() if math.isinf(norm_type) else torch.linalg.vector_norm(x, norm_type) ** norm_type)
    if not buckets:
        return torch.zeros(())
    parts = []
    for g, vals in buckets.values():
        v = torch.stack(vals).max() if math.isinf(norm_type) else torch.stack(vals).sum()
        if g is not None and dist.get_world_size(g) > 1:
            dist.all_reduce(v, op=dist.ReduceOp.MAX if math.isinf(norm_type) else dist.ReduceOp.SUM, group=g)
        parts.append(v)
    total = torch.stack(parts).max() if math.isinf(norm_type) else torch.stack(parts).sum() ** (1.0 / norm_type)
    if error_if_nonfinite and not torch.isfinite(total):
        raise RuntimeError(f"The total norm of order {norm_type} is non-finite, so it cannot be clipped.")
    return total


@torch.no_grad()
def compute_grad_norm_(parameters, norm_type: float = 2.0, error_if_nonfinite: bool = False, foreach=None):
    return compute_norm_(list(parameters), norm_type, error_if_nonfinite, foreach, grad=True)


@torch.no_grad()
def compute_param_norm_(parameters, norm_type: float = 2.0, error_if_nonfinite: bool = False, foreach=None):
    return compute_norm_(list(parameters), norm_type, error_if_nonfinite, foreach, grad=False)


@torch.no_grad()
def compute_single_param_std_(parameter: torch.Tensor) -> torch.Tensor:
    """Unbiased standard deviation of all elements of a (possibly distributed) parameter."""
    x = parameter.full_tensor() if hasattr(parameter, "full_tensor") else parameter
    x = x.detach().float()
    return (torch.sum(torch.square(x - x.mean())) / (x.numel() - 1)) ** 0.5


@torch.no_grad()
def clip_grad_norm_(parameters, max_norm: float, norm_type: float = 2.0, error_if_nonfinite: bool = False,
                    foreach=None) -> torch.Tensor:
    """Scales all gradients by ``min(1, max_norm / (total + 1e-6))``; returns the total norm before clipping."""
    parameters = [parameters] if isinstance(parameters, torch.Tensor) else list(parameters)
    total = compute_grad_norm_(parameters, norm_type, error_if_nonfinite, foreach)
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for p in parameters:
        if p.grad is not None:
            g = _local(p.grad)
            g.mul_(coef.to(device=g.device, dtype=g.dtype))
    return total
