"""Prototype (M6-T) gating of the legacy ``MOELayer``: logits ``[S tokens, Z prototypes, E experts]``, every prototype
routes independently, experts take at most ``capacity`` tokens per prototype and choice rank.

``topk_gating(logits, k, capacity, need_l_aux, dispatchV2)`` and ``switch_gating(logits, capacity, need_l_aux,
dispatchV2)`` return ``(l_aux, combine_weights [S, Z, E, C], dispatch_mask)`` or, with ``dispatchV2``, the compact form
``(l_aux, weights, (dispatch_idx [.., 2] = (expert, slot), E, C))`` whose k choices are concatenated along dim 0.

Rules (all per prototype): choice 1 is the arg-max of the softmax; choice c > 1 is the arg-max of the logits with the
*kept* earlier choices removed (a token whose earlier choice was dropped for capacity may pick that expert again);
slots are handed out in token order, choice rank by choice rank, after the slots of the earlier ranks; a choice
beyond ``capacity`` is dropped (weight 0, expert index 0); kept gate values are renormalised to sum to one per token;
the auxiliary loss is ``mean(mean_s(gates) * mean_s(first-choice one-hot))`` before dropping. Default capacity:
``ceil(1.25 S / E)``.
(Reference: atorch/modules/moe/topk_gating.py:11-165, switch_gating.py:24-190.)
"""
from __future__ import annotations

import math
from typing import List, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def _route(logits: torch.Tensor, k: int, capacity: int, need_l_aux: bool):
    gates = F.softmax(logits, dim=-1, dtype=torch.float).to(logits.dtype)          # [S, Z, E]
    S, Z, E = gates.shape
    cap = math.ceil(1.25 * S / E) if capacity < 0 else capacity
    remaining = logits
    taken = torch.zeros(1, Z, E, dtype=torch.long, device=logits.device)            # slots used by earlier ranks
    l_aux = torch.zeros((), device=logits.device)
    choices: List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]] = []
    for c in range(k):
        idx = torch.argmax(gates if c == 0 else remaining, dim=-1)                 # [S, Z]
        hot = F.one_hot(idx, E)                                                     # [S, Z, E]
        if c == 0 and need_l_aux:
            l_aux = (gates.mean(0) * hot.float().mean(0)).mean()
        slot = torch.cumsum(hot, 0) - 1 + taken
        kept = hot * (slot < cap)
        taken = taken + kept.sum(0, keepdim=True)
        alive = kept.sum(-1)                                                        # [S, Z] 1 if the choice survived
        choices.append(((gates * kept).sum(-1), idx * alive, (slot * kept).sum(-1), kept))
        remaining = remaining.masked_fill(kept.bool(), float("-inf"))
    denom = sum(g for g, _, _, _ in choices)
    denom = denom.clamp(min=torch.finfo(denom.dtype).eps)
    return gates, choices, denom, l_aux.to(logits.dtype), E, cap


def topk_gating(logits: torch.Tensor, k: int = 2, capacity: int = -1, need_l_aux: bool = False, dispatchV2: bool = False):
    gates, choices, denom, l_aux, E, cap = _route(logits, k, capacity, need_l_aux)
    if dispatchV2:
        weight = torch.cat([(g / denom).to(logits.dtype) for g, _, _, _ in choices], 0)
        where = torch.cat([torch.stack([e, s], -1) for _, e, s, _ in choices], 0)
        return l_aux, weight, (where, E, cap)
    combine = 0.0
    for g, _, s, kept in choices:
        w = (g / denom).unsqueeze(-1) * kept                                        # [S, Z, E]
        combine = combine + w.unsqueeze(3) * F.one_hot(s, cap).unsqueeze(2)
    return l_aux, combine.to(logits.dtype), combine.bool()


def switch_gating(logits: torch.Tensor, capacity: int = -1, need_l_aux: bool = False, dispatchV2: bool = False):
    """Top-1 form: the gate value itself is the weight (no renormalisation)."""
    gates, choices, _, l_aux, E, cap = _route(logits, 1, capacity, need_l_aux)
    g, e, s, kept = choices[0]
    if dispatchV2:
        return l_aux, g.to(logits.dtype), (torch.stack([e, s], -1), E, cap)
    combine = (gates * kept).unsqueeze(3) * F.one_hot(s, cap).unsqueeze(2)
    return l_aux, combine.to(logits.dtype), combine.bool()


class PrototypeTopkGate(nn.Module):
    """``l_aux, combine_weights, dispatch_mask = gate(input [S, M], bs, prototypes)``."""

    def __init__(self, model_dim: int, num_experts: int, k: int = 2, capacity: int = -1, need_l_aux: bool = False):
        super().__init__()
        self.wg = nn.Linear(model_dim, num_experts, bias=False)
        self.k, self.capacity, self.need_l_aux = k, capacity, need_l_aux

    def forward(self, input, bs=None, prototypes: int = 1, outer_batch: bool = False, dispatchV2: bool = False):
        if outer_batch:
            raise NotImplementedError("outer-batch routing is not implemented for the top-k gate")
        logits = self.wg(input).reshape(input.shape[0], prototypes, -1)
        return topk_gating(logits, self.k, self.capacity, self.need_l_aux, dispatchV2)


class PrototypeSwitchGate(nn.Module):
    def __init__(self, model_dim: int, num_experts: int, capacity: int = -1, need_l_aux: bool = False):
        super().__init__()
        self.wg = nn.Linear(model_dim, num_experts, bias=False)
        self.capacity, self.need_l_aux = capacity, need_l_aux

    def forward(self, input, bs=None, prototypes: int = 1, outer_batch: bool = False, dispatchV2: bool = False):
        if outer_batch:
            raise NotImplementedError("outer-batch routing is not implemented here")
        logits = self.wg(input).reshape(input.shape[0], prototypes, -1)
        return switch_gating(logits, self.capacity, self.need_l_aux, dispatchV2)


# names under which the reference's modules export them (atorch.modules.moe.topk_gating / switch_gating)
TopkGate = PrototypeTopkGate
SwitchGate = PrototypeSwitchGate
