"""``DistributedSelfAttention``: exact softmax attention with K/V sharded along the sequence and Q
processed in micro-chunks.

Per micro-chunk of queries: all-gather the chunk (``AllGatherQMicro``), local scores against this
rank's keys, ``DistributedSoftmax`` (all-reduce MAX then all-reduce SUM of the row statistics),
local context, ``ReduceScatterContext`` back to the owner of each query. Memory per rank is
O(S * S / sp); each micro step is checkpointed so only one chunk's scores live at a time.
(Reference: atorch/modules/distributed_transformer/distributed_attention.py:22-312, commu_utils.py:6-86.)
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ...modules.distributed_modules.mappings import all_gather_from_group, reduce_scatter_to_group
from ...utils.checkpoint import checkpoint_function


class _AllReduceMaxNoGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, op=dist.ReduceOp.MAX, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return None, None


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def distributed_softmax(scores: torch.Tensor, group) -> torch.Tensor:
    """Softmax over the last dim when that dim is sharded across ``group``."""
    m = _AllReduceMaxNoGrad.apply(scores.detach().amax(-1, keepdim=True), group)
    e = torch.exp(scores - m)
    z = _AllReduceSum.apply(e.sum(-1, keepdim=True), group)
    return e / z


class DistributedSelfAttention(nn.Module):
    """q, k, v: ``[B, H, S_local, D]`` (sequence-sharded); returns ``[B, H, S_local, D]``."""

    def __init__(self, num_micro_q: int = 1, group=None, softmax_scale: Optional[float] = None,
                 attention_dropout: float = 0.0):
        super().__init__()
        self.num_micro_q, self.group, self.softmax_scale = num_micro_q, group, softmax_scale
        self.dropout = nn.Dropout(attention_dropout)

    def set_sp(self, sp_size: int, sp_rank: int, sp_group) -> None:
        self.group = sp_group

    def _micro(self, q_chunk, k, v, scale):
        qg = all_gather_from_group(q_chunk, self.group, dim=2)               # [B, H, sp * q_micro, D]
        s = torch.matmul(qg, k.transpose(-1, -2)) * scale                      # local keys only
        p = self.dropout(distributed_softmax(s.float(), self.group).to(v.dtype))
        ctx = torch.matmul(p, v)                                               # partial sums over local keys
        return reduce_scatter_to_group(ctx, self.group, dim=2)                 # back to the query owners

    def forward(self, q, k, v, attention_mask=None):
        scale = self.softmax_scale if self.softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
        outs = []
        for qc in q.chunk(self.num_micro_q, dim=2):
            if torch.is_grad_enabled() and self.num_micro_q > 1:
                outs.append(checkpoint_function(self._micro, qc, k, v, scale))
            else:
                outs.append(self._micro(qc, k, v, scale))
        return torch.cat(outs, dim=2)
