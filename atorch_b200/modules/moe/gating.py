"""Routers: ``TopkGate`` (GShard-style top-k with capacity and auxiliary load-balancing loss),
``SwitchGate`` (top-1 with jitter and capacity) and ``TopNRouter`` (dropless top-k softmax with aux and
z losses, the router of the Mixtral-style examples).

Capacity: ``ceil(capacity_factor * tokens / experts)`` (at least ``min_capacity``); tokens beyond an
expert's capacity are dropped in arrival order. ``TopkGate.forward`` returns
``(l_aux, combine_weights [T, E, C], dispatch_mask [T, E, C], exp_counts)``.
(Reference: atorch/modules/moe/topk_gating.py:11-154, switch_gating.py:25-195,
examples/moe/moe_modules.py:57-112.)
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def _capacity(num_tokens: int, num_experts: int, capacity_factor: float, min_capacity: int) -> int:
    return max(int(math.ceil(capacity_factor * num_tokens / num_experts)), min_capacity)


def topk_gating(logits: torch.Tensor, k: int, capacity_factor: float, min_capacity: int = 4):
    T, E = logits.shape
    gates = F.softmax(logits.float(), dim=1)
    C = _capacity(T, E, capacity_factor * k, min_capacity)
    topv, topi = gates.topk(k, dim=1)                                  # [T, k]
    masks = F.one_hot(topi, E)                                         # [T, k, E]
    # auxiliary loss on the first choice (GShard)
    me, ce = gates.mean(0), masks[:, 0].float().mean(0)
    l_aux = (me * ce).sum() * E
    exp_counts = masks.sum((0, 1))
    # position of every (token, choice) inside its expert: choices are ranked choice-major
    flat = masks.permute(1, 0, 2).reshape(k * T, E)                    # choice 0 of all tokens first
    loc = torch.cumsum(flat, 0) - flat
    keep = (loc < C) & flat.bool()
    pos = (loc * flat).sum(1)                                          # [k*T]
    keep_tok = keep.any(1).view(k, T).t()                              # [T, k]
    pos = pos.view(k, T).t()
    w = topv * keep_tok
    w = w / w.sum(1, keepdim=True).clamp(min=torch.finfo(w.dtype).eps)
    combine = torch.zeros(T, E, C, dtype=gates.dtype, device=logits.device)
    t_idx = torch.arange(T, device=logits.device).unsqueeze(1).expand(T, k)
    sel = keep_tok
    combine[t_idx[sel], topi[sel], pos[sel]] = w[sel]
    return l_aux, combine.to(logits.dtype), combine.bool(), exp_counts


class TopkGate(nn.Module):
    def __init__(self, model_dim: int, num_experts: int, k: int = 2, capacity_factor: float = 1.0,
                 eval_capacity_factor: float = 1.0, min_capacity: int = 4, noisy_gate_policy: Optional[str] = None):
        super().__init__()
        self.wg = nn.Linear(model_dim, num_experts, bias=False)
        self.k, self.capacity_factor, self.eval_capacity_factor = k, capacity_factor, eval_capacity_factor
        self.min_capacity, self.noisy_gate_policy = min_capacity, noisy_gate_policy

    def forward(self, x: torch.Tensor):
        logits = self.wg(x.float() if self.wg.weight.dtype == torch.float32 else x)
        if self.noisy_gate_policy == "Jitter" and self.training:
            logits = logits * torch.empty_like(logits).uniform_(0.99, 1.01)
        cf = self.capacity_factor if self.training else self.eval_capacity_factor
        return topk_gating(logits, self.k, cf, self.min_capacity)


class SwitchGate(nn.Module):
    """Top-1 gate of Switch Transformer: multiplicative jitter on the input, capacity dropping, aux loss."""

    def __init__(self, model_dim: int, num_experts: int, capacity_factor: float = 1.0,
                 eval_capacity_factor: float = 1.0, min_capacity: int = 4, jitter_eps: float = 0.0):
        super().__init__()
        self.wg = nn.Linear(model_dim, num_experts, bias=False)
        self.capacity_factor, self.eval_capacity_factor = capacity_factor, eval_capacity_factor
        self.min_capacity, self.jitter_eps = min_capacity, jitter_eps

    def forward(self, x: torch.Tensor):
        if self.training and self.jitter_eps > 0:
            x = x * torch.empty_like(x).uniform_(1.0 - self.jitter_eps, 1.0 + self.jitter_eps)
        cf = self.capacity_factor if self.training else self.eval_capacity_factor
        return topk_gating(self.wg(x), 1, cf, self.min_capacity)


class TopNRouter(nn.Module):
    """Dropless top-k softmax router: returns ``(probs [T, k], indices [T, k])`` and keeps the auxiliary
    load-balancing loss and the router z-loss of the last call in ``self.aux_loss`` / ``self.z_loss``."""

    def __init__(self, hidden_size: int, num_experts: int, topk: int = 2, norm_prob: bool = True,
                 aux_loss_coef: float = 0.0, z_loss_coef: float = 0.0):
        super().__init__()
        self.classifier = nn.Linear(hidden_size, num_experts, bias=False)
        self.num_experts, self.topk, self.norm_prob = num_experts, topk, norm_prob
        self.aux_loss_coef, self.z_loss_coef = aux_loss_coef, z_loss_coef
        self.aux_loss = self.z_loss = None

    def forward(self, hidden_states: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        x = hidden_states.reshape(-1, hidden_states.shape[-1])
        logits = self.classifier(x).float()
        probs = F.softmax(logits, dim=-1)
        topv, topi = probs.topk(self.topk, dim=-1)
        if self.norm_prob:
            topv = topv / topv.sum(-1, keepdim=True)
        if self.aux_loss_coef > 0:
            frac = F.one_hot(topi, self.num_experts).float().sum(1).mean(0) / self.topk
            self.aux_loss = self.aux_loss_coef * self.num_experts * (frac * probs.mean(0)).sum()
        if self.z_loss_coef > 0:
            self.z_loss = self.z_loss_coef * torch.logsumexp(logits, dim=-1).pow(2).mean()
        return topv.to(hidden_states.dtype), topi
