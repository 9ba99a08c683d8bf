"""The PPO step functions with the list-based calling convention of the RLHF trainer: per-sample response slices
for the KL penalty and log-probabilities, rewards as a list of tensors, and a loss that takes its coefficients from a
config object and returns nested statistics. ``ppo_utils.py`` holds the batched, mask-based forms the trainer of this
package uses; both compute the same quantities.
(Reference: atorch/rl/ppo_utils/ppo_util.py:6-180.)
"""
from __future__ import annotations

import torch

from .model_util import get_tensor_stats, whiten
from .ppo_utils import logprobs_of_labels


def dist_fn(p: torch.Tensor) -> torch.distributions.Categorical:
    return torch.distributions.Categorical(logits=p)


def get_kl_penalty(logits, ref_logits, samples, glm_generation_inputs, attention_mask, kl_controller_value):
    """``samples`` = prompt | response tokens, ``glm_generation_inputs.input_ids`` = the (padded) prompts. Returns
    per-sample response slices of the log-probabilities and of ``-kl_coef * log_ratio``, the mean of the k3 KL
    estimator ``exp(r) - 1 - r`` and two scalars for logging."""
    logprobs = logprobs_of_labels(logits[:, :-1, :], samples[:, 1:])
    ref_logprobs = logprobs_of_labels(ref_logits[:, :-1, :], samples[:, 1:])
    start = glm_generation_inputs.input_ids.shape[1] - 1
    ends = start + attention_mask[:, start:].sum(1)
    log_ratio = (logprobs - ref_logprobs) * attention_mask[:, :-1]
    mean_kl = (log_ratio.exp() - 1 - log_ratio).mean()
    kl_penalty = kl_controller_value * -log_ratio
    stats = {"policy/mean_log_ratio": log_ratio.mean().item(), "policy/mean_kl_penalty": kl_penalty.mean().item()}
    n = samples.shape[0]
    return ([logprobs[i, start: ends[i]] for i in range(n)], [kl_penalty[i, start: ends[i]] for i in range(n)],
            mean_kl, stats)


def get_rewards(kl_penalty, scores, logprobs):
    """Per-sample rewards: the KL penalty slice with the sequence score added on its last token (in place); samples
    with an empty response are dropped."""
    rewards = []
    for i in range(scores.shape[0]):
        if len(kl_penalty[i]) == 0 or len(logprobs[i]) == 0:
            continue
        r = kl_penalty[i]
        r[-1] += scores[i]
        rewards.append(r)
    return rewards


def loss(logprobs, values, old_logprobs, old_values, advantages, returns, mask, logits, config=None):
    """Clipped PPO objective ``pg + vf_coef * vf - ent_coef * entropy`` over the masked tokens. ``config`` supplies
    ``clip_ratio`` (clamp the ratio itself before both surrogate terms), ``cliprange``, ``cliprange_value``,
    ``vf_coef``, ``ent_coef``."""
    cr, crv = config.cliprange, config.cliprange_value
    n = mask.sum()
    v_clipped = torch.clamp(values, old_values - crv, old_values + crv)
    vf1, vf2 = (values - returns) ** 2, (v_clipped - returns) ** 2
    vf_loss = 0.5 * torch.sum(torch.max(vf1, vf2) * mask) / n
    vf_clipfrac = torch.sum((vf2 > vf1).float() * mask) / n
    log_ratio = (logprobs - old_logprobs) * mask
    ratio = torch.exp(log_ratio)
    if config.clip_ratio:
        ratio = torch.clamp(ratio, 1.0 - cr, 1.0 + cr)
    with torch.no_grad():
        approx_kl = torch.mean((ratio - 1) - log_ratio)
    pg1, pg2 = -advantages * ratio, -advantages * torch.clamp(ratio, 1.0 - cr, 1.0 + cr)
    pg_loss = torch.sum(torch.max(pg1, pg2) * mask) / n
    pg_clipfrac = torch.sum((pg2 > pg1).float() * mask) / n
    ent_loss = torch.sum(dist_fn(logits).entropy() * mask) / n
    total = pg_loss + config.vf_coef * vf_loss - config.ent_coef * ent_loss
    stats = dict(
        losses=dict(total_loss=total.item(), policy_loss=pg_loss.item(), value_loss=vf_loss.item(),
                    entropy_loss=ent_loss.item()),
        values=dict(get_tensor_stats(values, mask, n), values_error=(torch.sum(((values - returns) * mask) ** 2) / n).item(),
                    clipfrac=vf_clipfrac.item()),
        old_values=get_tensor_stats(old_values, mask, n),
        returns=get_tensor_stats(returns, mask, n),
        policy=dict(approx_kl=approx_kl.item(), clipfrac=pg_clipfrac.item()),
        ratio=((ratio * mask).sum() / n).item(),
        padding_percentage=(n / mask.numel()).item(),
    )
    return total, stats


def get_advantages_and_returns(values, rewards, response_length, use_whitening=True, config=None):
    """Generalised advantage estimation over ``response_length`` steps (``config.gamma``, ``config.lam``), no mask:
    ``delta_t = r_t + gamma V_{t+1} - V_t``, ``A_t = delta_t + gamma lam A_{t+1}``; returns ``A + V``."""
    gamma, lam = config.gamma, config.lam
    running = 0
    adv = [None] * response_length
    for t in range(response_length - 1, -1, -1):
        next_v = values[:, t + 1] if t < response_length - 1 else 0.0
        running = rewards[:, t] + gamma * next_v - values[:, t] + gamma * lam * running
        adv[t] = running
    advantages = torch.stack(adv, dim=1)
    returns = advantages + values
    if use_whitening:
        advantages = whiten(advantages)
    return advantages.detach(), returns
