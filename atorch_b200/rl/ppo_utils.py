"""PPO numerics for RLHF: log-probabilities of labels, KL-penalised per-token rewards, generalised
advantage estimation (``delta_t = r_t + gamma V_{t+1} - V_t``, ``A_t = delta_t + gamma lambda A_{t+1}``),
clipped policy / value losses with an entropy bonus.
(Reference: atorch/rl/ppo_utils/ppo_util.py:19-180.)"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def logprobs_of_labels(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return torch.gather(F.log_softmax(logits.float(), dim=-1), -1, labels.unsqueeze(-1)).squeeze(-1)


def whiten(x: torch.Tensor, mask: Optional[torch.Tensor] = None, shift_mean: bool = True) -> torch.Tensor:
    if mask is None:
        mean, var = x.mean(), x.var(unbiased=False)
    else:
        n = mask.sum().clamp(min=1)
        mean = (x * mask).sum() / n
        var = ((x - mean) ** 2 * mask).sum() / n
    w = (x - mean) * torch.rsqrt(var + 1e-8)
    return w if shift_mean else w + mean


def compute_rewards(scores: torch.Tensor, logprobs: torch.Tensor, ref_logprobs: torch.Tensor, mask: torch.Tensor,
                    kl_coef: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token rewards: ``-kl_coef * (logp - logp_ref)`` everywhere, plus the sequence score on the last
    response token. Returns (rewards [B, T], mean KL)."""
    kl = (logprobs - ref_logprobs) * mask
    rewards = -kl_coef * kl
    last = (mask.cumsum(1) == mask.sum(1, keepdim=True)) & mask.bool()
    rewards = rewards + last.float() * scores.unsqueeze(1)
    return rewards, kl.sum(1).mean()


def gae(values: torch.Tensor, rewards: torch.Tensor, mask: torch.Tensor, gamma: float = 1.0, lam: float = 0.95,
        use_whitening: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    T = rewards.shape[1]
    adv = torch.zeros_like(rewards)
    last = torch.zeros(rewards.shape[0], device=rewards.device, dtype=rewards.dtype)
    for t in reversed(range(T)):
        nv = values[:, t + 1] if t + 1 < T else torch.zeros_like(last)
        delta = rewards[:, t] + gamma * nv * (mask[:, t + 1] if t + 1 < T else 0) - values[:, t]
        last = delta + gamma * lam * last * (mask[:, t + 1] if t + 1 < T else 0)
        adv[:, t] = last
    returns = adv + values
    if use_whitening:
        adv = whiten(adv, mask)
    return (adv * mask).detach(), (returns * mask).detach()


def ppo_loss(logprobs, values, old_logprobs, old_values, advantages, returns, mask, logits=None, cliprange=0.2,
             cliprange_value=0.2, vf_coef=0.5, ent_coef=0.0):
    n = mask.sum().clamp(min=1)
    vclip = old_values + (values - old_values).clamp(-cliprange_value, cliprange_value)
    vf_loss = 0.5 * (torch.max((values - returns) ** 2, (vclip - returns) ** 2) * mask).sum() / n
    ratio = torch.exp((logprobs - old_logprobs) * mask)
    pg = torch.max(-advantages * ratio, -advantages * ratio.clamp(1 - cliprange, 1 + cliprange))
    pg_loss = (pg * mask).sum() / n
    ent = torch.zeros((), device=logprobs.device)
    if logits is not None and ent_coef:
        p = F.softmax(logits.float(), -1)
        ent = (-(p * torch.log(p.clamp(min=1e-12))).sum(-1) * mask).sum() / n
    loss = pg_loss + vf_coef * vf_loss - ent_coef * ent
    stats = {"policy_loss": pg_loss.detach(), "value_loss": vf_loss.detach(), "entropy": ent.detach(),
             "clipfrac": (((ratio - 1).abs() > cliprange).float() * mask).sum() / n}
    return loss, stats
