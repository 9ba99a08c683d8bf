"""Softmax cross-entropy (label smoothing, z-loss, ignore_index, vocabulary-parallel) on the
sm_100a row kernels.

Reference counterparts: ``AtorchCrossEntropyLoss`` (atorch/modules/transformer/cross_entropy.py:7-71)
on the Triton kernels of atorch/kernels/triton_jit/cross_entropy.py:33-254, and
``vocab_parallel_cross_entropy`` (atorch/modules/distributed_modules/cross_entropy.py:9-127).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib


def cross_entropy_reference(logits, labels, ignore_index=-100, label_smoothing=0.0, lse_square_scale=0.0):
    """Per-row loss in fp32 (0 for ignored rows)."""
    lf = logits.float()
    loss = torch.nn.functional.cross_entropy(lf, labels, ignore_index=ignore_index, reduction="none",
                                             label_smoothing=label_smoothing)
    if lse_square_scale:
        lse = torch.logsumexp(lf, dim=-1)
        loss = loss + torch.where(labels == ignore_index, torch.zeros_like(lse), lse_square_scale * lse * lse)
    return loss


def _fwd_launch(logits, labels, loss, lse, label_logit, sum_logits, vocab_start, v_total, ignore_index, smoothing, z):
    rows, V = logits.shape
    rc = _lib.lib().atb_ce_fwd(_lib.ptr(logits), _lib.ptr(labels), _lib.ptr(loss), _lib.ptr(lse),
                               _lib.ptr(label_logit), _lib.ptr(sum_logits), ctypes.c_longlong(rows), ctypes.c_int(V),
                               ctypes.c_longlong(logits.stride(0)), ctypes.c_int(vocab_start),
                               ctypes.c_longlong(v_total), ctypes.c_longlong(ignore_index),
                               ctypes.c_float(smoothing), ctypes.c_float(z), ctypes.c_int(_lib.DT[logits.dtype]),
                               _lib.stream_ptr())
    _lib.check(rc, "atb_ce_fwd")


def _bwd_launch(logits, labels, lse, dloss, dlogits, vocab_start, v_total, ignore_index, smoothing, z):
    rows, V = logits.shape
    rc = _lib.lib().atb_ce_bwd(_lib.ptr(logits), _lib.ptr(labels), _lib.ptr(lse), _lib.ptr(dloss),
                               ctypes.c_float(1.0), _lib.ptr(dlogits), ctypes.c_longlong(rows), ctypes.c_int(V),
                               ctypes.c_longlong(logits.stride(0)), ctypes.c_int(vocab_start),
                               ctypes.c_longlong(v_total), ctypes.c_longlong(ignore_index),
                               ctypes.c_float(smoothing), ctypes.c_float(z), ctypes.c_int(_lib.DT[logits.dtype]),
                               _lib.stream_ptr())
    _lib.check(rc, "atb_ce_bwd")


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index, smoothing, z, inplace_backward, group):
        rows, V = logits.shape
        dev = logits.device
        loss = torch.empty(rows, dtype=torch.float32, device=dev)
        lse = torch.empty(rows, dtype=torch.float32, device=dev)
        world = dist.get_world_size(group) if group is not None else 1
        if world == 1:
            _fwd_launch(logits, labels, loss, lse, None, None, 0, V, ignore_index, smoothing, z)
            vocab_start, v_total = 0, V
        else:
            rank = dist.get_rank(group)
            vocab_start, v_total = rank * V, V * world
            ll = torch.empty(rows, dtype=torch.float32, device=dev)
            tot = torch.empty(rows, dtype=torch.float32, device=dev)
            _fwd_launch(logits, labels, None, lse, ll, tot, vocab_start, v_total, ignore_index, smoothing, z)
            all_lse = torch.empty(world, rows, dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(all_lse, lse, group=group)
            lse = torch.logsumexp(all_lse, dim=0)
            packed = torch.stack([ll, tot])
            dist.all_reduce(packed, group=group)
            ll, tot = packed[0], packed[1]
            valid = labels != ignore_index
            loss = (lse - ll) * (1.0 - smoothing)
            if smoothing > 0:
                loss = loss + smoothing * (lse - tot / v_total)
            loss = loss + z * lse * lse
            loss = torch.where(valid, loss, torch.zeros_like(loss))
        ctx.save_for_backward(logits, labels, lse)
        ctx.cfg = (vocab_start, v_total, ignore_index, smoothing, z, inplace_backward)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, labels, lse = ctx.saved_tensors
        vocab_start, v_total, ignore_index, smoothing, z, inplace = ctx.cfg
        dlogits = logits if inplace else torch.empty_strided(logits.shape, logits.stride(), dtype=logits.dtype,
                                                              device=logits.device)
        _bwd_launch(logits, labels, lse, dloss.contiguous().float(), dlogits, vocab_start, v_total, ignore_index,
                    smoothing, z)
        return dlogits, None, None, None, None, None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, label_smoothing: float = 0.0,
                  lse_square_scale: float = 0.0, inplace_backward: bool = False,
                  process_group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Per-row losses ``[rows]`` (fp32). With ``process_group`` the vocabulary is split across the
    group (rank r holds columns ``[r*V, (r+1)*V)``) and labels are global ids."""
    assert logits.dim() == 2 and labels.dim() == 1
    ok = (_lib.use_kernels(logits) and logits.dtype in (torch.bfloat16, torch.float32)
          and logits.stride(1) == 1 and logits.stride(0) % 8 == 0)
    if not ok:
        if process_group is not None and dist.get_world_size(process_group) > 1:
            return _vocab_parallel_reference(logits, labels, ignore_index, label_smoothing, lse_square_scale,
                                             process_group)
        return cross_entropy_reference(logits, labels, ignore_index, label_smoothing, lse_square_scale)
    return _CrossEntropy.apply(logits, labels.contiguous(), ignore_index, float(label_smoothing),
                               float(lse_square_scale), inplace_backward, process_group)


class _VocabParallelRef(torch.autograd.Function):
    """PyTorch evaluation of the vocabulary-parallel loss (CPU / oracle path). The forward combines
    the ranks' pieces with all-reduces; the backward is purely local, like the kernel's:
    ``dlogits = dloss * (p (1 + 2 z lse) - (1 - eps) onehot - eps / V)`` on this rank's slice."""

    @staticmethod
    def forward(ctx, logits, labels, ignore_index, smoothing, z, group):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        V = logits.shape[1]
        lf = logits.float()
        gmax = lf.max(dim=-1).values
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
        sumexp = (lf - gmax[:, None]).exp().sum(-1)
        dist.all_reduce(sumexp, group=group)
        lse = gmax + sumexp.log()
        local = labels - rank * V
        inside = (local >= 0) & (local < V) & (labels != ignore_index)
        ll = torch.where(inside, lf.gather(1, local.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(lse))
        tot = lf.sum(-1)
        packed = torch.stack([ll, tot])
        dist.all_reduce(packed, group=group)
        ll, tot = packed[0], packed[1]
        loss = (lse - ll) * (1.0 - smoothing)
        if smoothing > 0:
            loss = loss + smoothing * (lse - tot / (V * world))
        loss = loss + z * lse * lse
        valid = labels != ignore_index
        ctx.save_for_backward(logits, lse, local, inside, valid)
        ctx.cfg = (smoothing, z, V * world)
        return torch.where(valid, loss, torch.zeros_like(loss))

    @staticmethod
    def backward(ctx, dloss):
        logits, lse, local, inside, valid = ctx.saved_tensors
        smoothing, z, v_total = ctx.cfg
        g = torch.where(valid, dloss.float(), torch.zeros_like(lse))
        p = (logits.float() - lse[:, None]).exp()
        d = p * (g * (1.0 + 2.0 * z * lse))[:, None] - (g * smoothing / v_total)[:, None]
        idx = local.clamp(0, logits.shape[1] - 1)[:, None]
        d.scatter_add_(1, idx, (-(g * (1.0 - smoothing)) * inside.float())[:, None])
        return d.to(logits.dtype), None, None, None, None, None


def _vocab_parallel_reference(logits, labels, ignore_index, smoothing, z, group):
    return _VocabParallelRef.apply(logits, labels, ignore_index, float(smoothing), float(z), group)
