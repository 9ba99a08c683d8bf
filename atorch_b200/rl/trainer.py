"""RLHF with PPO: config, replay buffer, model engine and trainer.

``ModelEngine`` holds actor / critic / reference / reward models; each is accelerated with its own
strategy inside its own ``ParallelGroupContextManager(model_type)`` so that the four models may use
different parallel layouts side by side. ``PPOTrainer.train`` loops: sample prompts -> ``make_experience``
(generate responses, score them, compute reference log-probs and values) until ``num_rollouts`` are
buffered -> ``ppo_epochs`` passes of clipped PPO updates -> clear the buffer.
(Reference: atorch/rl/config.py:22-280, model_engine/model_engine.py:39-500, trainer/rl_trainer.py:69-90,
replay_buffer/.)"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.nn as nn

from ..auto.accelerate import auto_accelerate
from ..distributed.distributed import ParallelGroupContextManager
from . import ppo_utils as P


@dataclass
class PPOConfig:
    ppo_epoch: int = 2
    num_rollouts: int = 16
    batch_size: int = 8
    init_kl_coef: float = 0.05
    gamma: float = 1.0
    lam: float = 0.95
    cliprange: float = 0.2
    cliprange_value: float = 0.2
    vf_coef: float = 0.5
    ent_coef: float = 0.0
    max_new_tokens: int = 8
    temperature: float = 1.0


@dataclass
class ModelSpec:
    model: Optional[nn.Module] = None
    train_strategy: Any = "torch_native"        # "torch_native" | list strategy for auto_accelerate
    optimizer_cls: Any = torch.optim.AdamW
    optimizer_args: Dict[str, Any] = field(default_factory=lambda: {"lr": 1e-4})
    trainable: bool = False


@dataclass
class AtorchRLConfig:
    actor: ModelSpec = field(default_factory=ModelSpec)
    critic: ModelSpec = field(default_factory=ModelSpec)
    ref_model: ModelSpec = field(default_factory=ModelSpec)
    reward_model: ModelSpec = field(default_factory=ModelSpec)
    ppo_config: PPOConfig = field(default_factory=PPOConfig)


class ReplayBuffer:
    def __init__(self):
        self.items: List[Dict[str, torch.Tensor]] = []

    @property
    def num(self) -> int:
        return sum(i["input_ids"].shape[0] for i in self.items)

    def add(self, sample: Dict[str, torch.Tensor]) -> None:
        self.items.append({k: v.detach() for k, v in sample.items()})

    def reset(self) -> None:
        self.items = []

    def batches(self, batch_size: int):
        cat = {k: torch.cat([i[k] for i in self.items]) for k in self.items[0]}
        n = cat["input_ids"].shape[0]
        perm = torch.randperm(n)
        for s in range(0, n, batch_size):
            idx = perm[s: s + batch_size]
            yield {k: v[idx] for k, v in cat.items()}


class ModelEngine:
    """States: ``init`` -> ``experience_generation`` <-> ``rl_training``."""

    def __init__(self, config: AtorchRLConfig):
        self.config, self.state = config, "init"
        self.models: Dict[str, nn.Module] = {}
        self.optims: Dict[str, Any] = {}
        for name in ("actor", "critic", "ref_model", "reward_model"):
            spec: ModelSpec = getattr(config, name)
            if spec.model is None:
                continue
            with ParallelGroupContextManager(name + "_"):
                if spec.train_strategy == "torch_native" or spec.train_strategy is None:
                    self.models[name] = spec.model
                    if spec.trainable:
                        self.optims[name] = spec.optimizer_cls(spec.model.parameters(), **spec.optimizer_args)
                else:
                    ok, res, _ = auto_accelerate(spec.model, spec.optimizer_cls if spec.trainable else None,
                                                 optim_args=spec.optimizer_args, load_strategy=spec.train_strategy,
                                                 ignore_dryrun_on_load_strategy=True, find_unused_parameters=True)
                    assert ok, f"could not accelerate the {name} model"
                    self.models[name], self.optims[name] = res.model, res.optim
            if not spec.trainable:
                for p in self.models[name].parameters():
                    p.requires_grad_(False)

    def set_state(self, state: str) -> None:
        assert state in ("experience_generation", "rl_training")
        self.state = state
        for n, m in self.models.items():
            m.train(state == "rl_training" and getattr(self.config, n).trainable)

    def save(self, path: str) -> None:
        torch.save({n: m.state_dict() for n, m in self.models.items() if getattr(self.config, n).trainable}, path)

    def load(self, path: str) -> None:
        for n, sd in torch.load(path).items():
            self.models[n].load_state_dict(sd)


class PPOTrainer:
    """Actor: ``actor(ids) -> logits [B, T, V]``; critic: ``critic(ids) -> values [B, T]``;
    reward model: ``reward(ids) -> scores [B]``."""

    def __init__(self, engine: ModelEngine, prompts: List[torch.Tensor], generate_fn: Optional[Callable] = None):
        self.engine, self.cfg, self.prompts = engine, engine.config.ppo_config, prompts
        self.buffer = ReplayBuffer()
        self.generate_fn = generate_fn or self._sample
        self.kl_coef = self.cfg.init_kl_coef
        self.log: List[Dict[str, float]] = []

    @torch.no_grad()
    def _sample(self, actor, prompt: torch.Tensor) -> torch.Tensor:
        ids = prompt
        for _ in range(self.cfg.max_new_tokens):
            logits = actor(ids)[:, -1].float() / self.cfg.temperature
            ids = torch.cat([ids, torch.multinomial(torch.softmax(logits, -1), 1)], dim=1)
        return ids

    @torch.no_grad()
    def make_experience(self, prompt: torch.Tensor) -> None:
        m = self.engine.models
        self.engine.set_state("experience_generation")
        ids = self.generate_fn(m["actor"], prompt)
        plen = prompt.shape[1]
        mask = torch.zeros(ids.shape, dtype=torch.float32)
        mask[:, plen:] = 1.0
        mask = mask[:, 1:]
        logp = P.logprobs_of_labels(m["actor"](ids)[:, :-1], ids[:, 1:])
        ref = P.logprobs_of_labels(m["ref_model"](ids)[:, :-1], ids[:, 1:])
        values = m["critic"](ids)[:, :-1].float()
        scores = m["reward_model"](ids).float()
        rewards, kl = P.compute_rewards(scores, logp, ref, mask, self.kl_coef)
        adv, ret = P.gae(values * mask, rewards, mask, self.cfg.gamma, self.cfg.lam)
        self.buffer.add(dict(input_ids=ids, mask=mask, logprobs=logp, values=values, advantages=adv, returns=ret))
        self.log.append({"score": scores.mean().item(), "kl": kl.item()})

    def rl_training(self) -> Dict[str, float]:
        m, o, c = self.engine.models, self.engine.optims, self.cfg
        self.engine.set_state("rl_training")
        stats = {}
        for _ in range(c.ppo_epoch):
            for b in self.buffer.batches(c.batch_size):
                logits = m["actor"](b["input_ids"])[:, :-1]
                logp = P.logprobs_of_labels(logits, b["input_ids"][:, 1:])
                values = m["critic"](b["input_ids"])[:, :-1].float()
                loss, stats = P.ppo_loss(logp, values, b["logprobs"], b["values"], b["advantages"], b["returns"],
                                         b["mask"], logits, c.cliprange, c.cliprange_value, c.vf_coef, c.ent_coef)
                for opt in o.values():
                    opt.zero_grad()
                loss.backward()
                for opt in o.values():
                    opt.step()
        return {k: float(v) for k, v in stats.items()}

    def train(self, iterations: int = 1) -> List[Dict[str, float]]:
        out = []
        for _ in range(iterations):
            i = 0
            while self.buffer.num < self.cfg.num_rollouts:
                self.make_experience(self.prompts[i % len(self.prompts)])
                i += 1
            out.append(self.rl_training())
            self.buffer.reset()
        return out
