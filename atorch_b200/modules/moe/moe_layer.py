"""``MOELayer`` / ``Experts``: capacity-based (GShard) mixture of experts.

Dispatch ``einsum("sec,sm->ecm")`` with the gate's mask, all-to-all over the expert group, local
experts, all-to-all back, combine ``einsum("sec,ecm->sm")``.
(Reference: atorch/modules/moe/moe_layer.py:22-611; expert-group registration
``set_experts_process_group`` and the DDP variant in atorch/modules/moe/ddp.py:31-360.)
"""
from __future__ import annotations

import copy
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ...communication.functions import all_to_all
from ...distributed import distributed as D

_EXPERTS_PG = {"group": None}


def set_experts_process_group(group) -> None:
    _EXPERTS_PG["group"] = group


def get_experts_process_group():
    return _EXPERTS_PG["group"] if _EXPERTS_PG["group"] is not None else D.parallel_group("expert")


class Experts(nn.Module):
    """``num_local_experts`` copies of an expert module applied to ``[E_local, C, M]`` chunks."""

    def __init__(self, expert: nn.Module, num_local_experts: int = 1):
        super().__init__()
        self.experts = nn.ModuleList([copy.deepcopy(expert) for _ in range(num_local_experts)])
        self.num_local_experts = num_local_experts
        for e in self.experts:
            for p in e.parameters():
                p.expert = True          # marks parameters that are not replicated over the data group

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        chunks = x.chunk(self.num_local_experts, dim=1)
        return torch.cat([e(c) for e, c in zip(self.experts, chunks)], dim=1)


class MOELayer(nn.Module):
    def __init__(self, gate: nn.Module, experts: Experts, num_local_experts: Optional[int] = None, group=None,
                 outer_batch: bool = False):
        super().__init__()
        self.gate, self.experts = gate, experts
        self.num_local_experts = num_local_experts or experts.num_local_experts
        self.group = group
        self.l_aux = None
        self.exp_counts = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        group = self.group if self.group is not None else get_experts_process_group()
        ep = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        shape = x.shape
        tokens = x.reshape(-1, shape[-1])
        self.l_aux, combine, mask, self.exp_counts = self.gate(tokens)
        dispatched = torch.einsum("sec,sm->ecm", mask.to(tokens.dtype), tokens)      # [E, C, M]
        E, C, M = dispatched.shape
        if ep > 1:
            dispatched = all_to_all(group, dispatched.contiguous())
        dispatched = dispatched.reshape(ep, self.num_local_experts, C, M)
        out = self.experts(dispatched)
        out = out.reshape(E, C, M)
        if ep > 1:
            out = all_to_all(group, out.contiguous())
        y = torch.einsum("sec,ecm->sm", combine.to(out.dtype), out)
        return y.view(shape)
