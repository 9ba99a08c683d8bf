"""Autograd collectives used by expert parallelism: all-to-all (equal or variable splits),
gather to / reduce-scatter from the MoE region.
(Reference: atorch/communication/functions.py:12-171.)
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _ws(g):
    return dist.get_world_size(g) if (dist.is_available() and dist.is_initialized()) else 1


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, x, output_split_sizes, input_split_sizes):
        ctx.group, ctx.out_splits, ctx.in_splits = group, output_split_sizes, input_split_sizes
        if _ws(group) == 1:
            return x
        x = x.contiguous()
        if output_split_sizes is None:
            out = torch.empty_like(x)
        else:
            out = x.new_empty((sum(output_split_sizes),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, output_split_sizes=output_split_sizes, input_split_sizes=input_split_sizes,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return None, _AllToAll.apply(ctx.group, g, ctx.in_splits, ctx.out_splits), None, None


def all_to_all(group, x: torch.Tensor, output_split_sizes: Optional[List[int]] = None,
               input_split_sizes: Optional[List[int]] = None) -> torch.Tensor:
    return _AllToAll.apply(group, x, output_split_sizes, input_split_sizes)


def _gather_dim0(x, group):
    w = _ws(group)
    if w == 1:
        return x
    x = x.contiguous()
    out = x.new_empty((w * x.shape[0],) + tuple(x.shape[1:]))
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def _reduce_scatter_dim0(x, group):
    w = _ws(group)
    if w == 1:
        return x
    x = x.contiguous()
    out = x.new_empty((x.shape[0] // w,) + tuple(x.shape[1:]))
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


class _GatherToMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim0(g, ctx.group), None


class _ReduceScatterFromMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return _gather_dim0(g, ctx.group), None


def gather_from_expert_parallel_region_to_moe(x, group):
    return _GatherToMoE.apply(x, group)


def reduce_scatter_to_expert_parallel_region_from_moe(x, group):
    return _ReduceScatterFromMoE.apply(x, group)
