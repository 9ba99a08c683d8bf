"""Autograd mappings between replicated and sharded tensors inside a tensor-parallel group.

    copy_to_group            fwd identity            bwd all-reduce
    reduce_from_group        fwd all-reduce          bwd identity
    scatter_to_group         fwd keep own chunk      bwd all-gather      (along ``dim``)
    gather_from_group        fwd all-gather          bwd keep own chunk
    reduce_scatter_to_group  fwd reduce-scatter      bwd all-gather      (sequence parallel exit)
    all_gather_from_group    fwd all-gather          bwd reduce-scatter  (sequence parallel entry)
    split_last_dim_gather_first_dim / its inverse: one all-to-all each
    collect_and_reshard      gather along one dim then split along another

(Reference: atorch/modules/distributed_modules/mappings.py:23-456.)
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _ws(group):
    return dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1


def _all_gather(x, dim, group):
    w = _ws(group)
    if w == 1:
        return x
    x = x.contiguous()
    out = torch.empty((w * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    if dim % x.dim() == 0:
        return out
    return torch.cat(list(out.view((w,) + tuple(x.shape)).unbind(0)), dim=dim)


def _split(x, dim, group):
    w = _ws(group)
    if w == 1:
        return x
    return x.chunk(w, dim=dim)[dist.get_rank(group)].contiguous()


def _reduce_scatter(x, dim, group):
    w = _ws(group)
    if w == 1:
        return x
    chunks = torch.cat([c.contiguous() for c in x.chunk(w, dim=dim)], dim=0)
    out = torch.empty((chunks.shape[0] // w,) + tuple(chunks.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, chunks, group=group)
    return out


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _ws(ctx.group) > 1:
            g = g.contiguous()
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        if _ws(group) > 1:
            x = x.contiguous().clone()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.cfg = (dim, group)
        return _split(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        dim, group = ctx.cfg
        return _all_gather(g, dim, group), None, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.cfg = (dim, group)
        return _all_gather(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        dim, group = ctx.cfg
        return _split(g, dim, group), None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.cfg = (dim, group)
        return _reduce_scatter(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        dim, group = ctx.cfg
        return _all_gather(g, dim, group), None, None


class _AllGatherRS(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.cfg = (dim, group)
        return _all_gather(x, dim, group)

    @staticmethod
    def backward(ctx, g):
        dim, group = ctx.cfg
        return _reduce_scatter(g, dim, group), None, None


class _A2A(torch.autograd.Function):
    """Split ``split_dim`` over the group and concatenate what arrives along ``cat_dim``."""

    @staticmethod
    def forward(ctx, x, split_dim, cat_dim, group):
        ctx.cfg = (split_dim, cat_dim, group)
        w = _ws(group)
        if w == 1:
            return x
        send = torch.stack([c.contiguous() for c in x.chunk(w, dim=split_dim)])
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return torch.cat(list(recv.unbind(0)), dim=cat_dim)

    @staticmethod
    def backward(ctx, g):
        split_dim, cat_dim, group = ctx.cfg
        return _A2A.apply(g, cat_dim, split_dim, group), None, None, None


def copy_to_group(x, group=None):
    return _Copy.apply(x, group)


def reduce_from_group(x, group=None):
    return _Reduce.apply(x, group)


def scatter_to_group(x, group=None, dim=-1):
    return _Scatter.apply(x, dim, group)


def gather_from_group(x, group=None, dim=-1):
    return _Gather.apply(x, dim, group)


def reduce_scatter_to_group(x, group=None, dim=0):
    return _ReduceScatter.apply(x, dim, group)


def all_gather_from_group(x, group=None, dim=0):
    return _AllGatherRS.apply(x, dim, group)


def split_last_dim_gather_first_dim(x, group=None):
    return _A2A.apply(x, x.dim() - 1, 0, group)


def split_first_dim_gather_last_dim(x, group=None):
    return _A2A.apply(x, 0, x.dim() - 1, group)


def collect_and_reshard(x, gather_dim, split_dim, group=None):
    return _Scatter.apply(_Gather.apply(x, gather_dim, group), split_dim, group)
