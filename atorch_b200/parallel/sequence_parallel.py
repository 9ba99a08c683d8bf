"""Long-context attention over a sequence-parallel group.

* ``UlyssesAttention``: every rank holds ``S / sp`` tokens outside attention; one all-to-all swaps to
  the full sequence with ``H / sp`` heads, attention runs locally (flash kernels), a second
  all-to-all swaps back. ``set_sp(sp_size, sp_rank, sp_group)`` is the hook called by the
  ``sequence_parallel`` optimisation.
* ``ring_attention``: on GPUs of one NVLink domain the flash kernels run per chunk and the copy engines pull the
  peers' K/V chunks out of symmetric memory (``ops/ring_flash.py``); elsewhere (CPU / gloo, odd shapes) K/V stay
  sequence-sharded and travel round the ring with dense attention per step (``sp - 1`` send/recv steps);
  each step's partial output is merged with the running one through the log-sum-exp rule
  ``o = (o1 e^{l1} + o2 e^{l2}) / (e^{l1} + e^{l2})``. Causal masking uses contiguous chunks: a rank
  skips chunks from higher ranks and runs the diagonal chunk causally. Differentiable through autograd.
(Reference: ``seq_all_to_all`` users in atorch/distributed/distributed.py:613-679; the reference has no
ring attention of its own, it only reaches context parallelism through Megatron.)
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..distributed.distributed import seq_all_to_all


class UlyssesAttention(nn.Module):
    """q, k, v: ``[B, S_local, H, D]`` -> ``[B, S_local, H, D]``."""

    def __init__(self, causal: bool = True, softmax_scale: Optional[float] = None, attention_dropout: float = 0.0):
        super().__init__()
        self.causal, self.softmax_scale, self.attention_dropout = causal, softmax_scale, attention_dropout
        self.sp_size, self.sp_rank, self.sp_group = 1, 0, None

    def set_sp(self, sp_size: int, sp_rank: int, sp_group) -> None:
        self.sp_size, self.sp_rank, self.sp_group = sp_size, sp_rank, sp_group

    def forward(self, q, k, v, **attn_kwargs):
        if self.sp_size > 1:
            q = seq_all_to_all(q, 2, 1, self.sp_group, self.sp_size)      # scatter heads, gather sequence
            k = seq_all_to_all(k, 2, 1, self.sp_group, self.sp_size)
            v = seq_all_to_all(v, 2, 1, self.sp_group, self.sp_size)
        o = ops.attention(q, k, v, causal=self.causal, softmax_scale=self.softmax_scale,
                          dropout_p=self.attention_dropout if self.training else 0.0, **attn_kwargs)
        if self.sp_size > 1:
            o = seq_all_to_all(o, 1, 2, self.sp_group, self.sp_size)      # scatter sequence, gather heads
        return o


def _attn_with_lse(q, k, v, causal: bool, scale: float):
    """Dense attention returning (out [B,S,H,D] fp32, lse [B,H,S]); used per ring step."""
    qf, kf, vf = q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2)
    if kf.shape[1] != qf.shape[1]:
        rep = qf.shape[1] // kf.shape[1]
        kf, vf = kf.repeat_interleave(rep, 1), vf.repeat_interleave(rep, 1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        Sq, Sk = s.shape[-2:]
        s = s.masked_fill(torch.ones(Sq, Sk, dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.softmax(s, dim=-1), vf)
    return o.transpose(1, 2), lse


class _RingExchange(torch.autograd.Function):
    """Send ``x`` to the next rank of the ring and receive from the previous one; the backward sends
    gradients the opposite way."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _ring_pass(x, group, +1)

    @staticmethod
    def backward(ctx, g):
        return _ring_pass(g.contiguous(), ctx.group, -1), None


def _ring_pass(x, group, direction: int):
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    dst = dist.get_global_rank(group, (rank + direction) % world) if group is not None else (rank + direction) % world
    src = dist.get_global_rank(group, (rank - direction) % world) if group is not None else (rank - direction) % world
    x = x.contiguous()
    out = torch.empty_like(x)
    reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, x, dst, group), dist.P2POp(dist.irecv, out, src, group)])
    for r in reqs:
        r.wait()
    return out


def ring_attention(q, k, v, group=None, causal: bool = True, softmax_scale: Optional[float] = None,
                   layout: str = "contiguous"):
    """q, k, v are this rank's part of the sequence ``[B, S/sp, H, D]``; returns that part's output.
    ``layout="contiguous"``: consecutive chunks in rank order. ``layout="zigzag"`` (GPU form only): parts made by
    ``ops.ring_flash.zigzag_shard``, which balances the causal work over the ranks."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if world > 1 and q.is_cuda:
        from ..ops import ring_flash

        grp = group if group is not None else dist.group.WORLD
        if ring_flash.available(q, k, v, grp):      # flash kernels per chunk, chunks pulled over peer memory
            return ring_flash.ring_flash_attention(q, k, v, grp, causal, scale, layout)
    if layout != "contiguous" and causal and world > 1:
        raise NotImplementedError("the zigzag layout needs the flash / peer-memory form (CUDA, bf16, head dim 64 or 128)")
    out, lse = None, None
    kv = torch.stack([k, v])
    for step in range(world):
        src = (rank - step) % world                     # whose K/V chunk we hold at this step
        if not causal or src <= rank:
            o_i, l_i = _attn_with_lse(q, kv[0], kv[1], causal and src == rank, scale)
            if out is None:
                out, lse = o_i, l_i
            else:
                new_lse = torch.logaddexp(lse, l_i)
                w_old = torch.exp(lse - new_lse).transpose(1, 2).unsqueeze(-1)
                w_new = torch.exp(l_i - new_lse).transpose(1, 2).unsqueeze(-1)
                out, lse = out * w_old + o_i * w_new, new_lse
        elif out is not None:
            # a skipped chunk must still sit in the autograd graph: its (zero) gradient has to travel
            # back round the ring, or the ranks that did use it would wait for a transfer that never starts
            out = out + (kv.float() * 0.0).sum()
        if step + 1 < world:
            kv = _RingExchange.apply(kv, group)
    return out.to(q.dtype)


class RingAttention(nn.Module):
    def __init__(self, causal: bool = True, softmax_scale: Optional[float] = None):
        super().__init__()
        self.causal, self.softmax_scale = causal, softmax_scale
        self.sp_group = None

    def set_sp(self, sp_size: int, sp_rank: int, sp_group) -> None:
        self.sp_group = sp_group

    def forward(self, q, k, v):
        return ring_attention(q, k, v, self.sp_group, self.causal, self.softmax_scale)
