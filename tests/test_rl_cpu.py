"""PPO utilities and a tiny end-to-end RLHF loop on CPU."""
import torch
import torch.nn as nn

from atorch_b200.rl import (AtorchRLConfig, ModelEngine, ModelSpec, PPOConfig, PPOTrainer, compute_rewards, gae,
                            logprobs_of_labels, ppo_loss)


def test_gae_matches_manual():
    values = torch.tensor([[0.5, 0.4, 0.3]])
    rewards = torch.tensor([[0.0, 0.0, 1.0]])
    mask = torch.ones(1, 3)
    adv, ret = gae(values, rewards, mask, gamma=1.0, lam=1.0, use_whitening=False)
    assert torch.allclose(adv, torch.tensor([[0.5, 0.6, 0.7]]), atol=1e-6)
    assert torch.allclose(ret, adv + values)
    r, kl = compute_rewards(torch.tensor([2.0]), torch.zeros(1, 3), torch.ones(1, 3) * 0.1,
                            torch.tensor([[0.0, 1.0, 1.0]]), kl_coef=0.5)
    assert torch.allclose(r, torch.tensor([[0.0, 0.05, 2.05]])) and abs(kl.item() + 0.2) < 1e-6
    lp = logprobs_of_labels(torch.zeros(1, 2, 4), torch.tensor([[1, 2]]))
    assert torch.allclose(lp, torch.full((1, 2), -1.3863), atol=1e-4)
    loss, st = ppo_loss(lp, values[:, :2], lp, values[:, :2], adv[:, :2], ret[:, :2], mask[:, :2])
    assert torch.isfinite(loss) and st["clipfrac"] == 0


class LM(nn.Module):
    def __init__(self, V=16, h=32):
        super().__init__()
        self.e, self.l, self.o = nn.Embedding(V, h), nn.Linear(h, h), nn.Linear(h, V)

    def forward(self, ids):
        return self.o(torch.tanh(self.l(self.e(ids))))


class Critic(LM):
    def forward(self, ids):
        return super().forward(ids).mean(-1)


class Reward(nn.Module):
    def forward(self, ids):                      # likes token 3
        return (ids == 3).float().mean(1) * 4.0


def test_ppo_loop_improves_reward():
    torch.manual_seed(0)
    actor = LM()
    ref = LM()
    ref.load_state_dict(actor.state_dict())
    cfg = AtorchRLConfig(actor=ModelSpec(actor, optimizer_args={"lr": 3e-3}, trainable=True),
                         critic=ModelSpec(Critic(), optimizer_args={"lr": 3e-3}, trainable=True),
                         ref_model=ModelSpec(ref), reward_model=ModelSpec(Reward()),
                         ppo_config=PPOConfig(num_rollouts=32, batch_size=16, ppo_epoch=2, init_kl_coef=0.01))
    eng = ModelEngine(cfg)
    tr = PPOTrainer(eng, [torch.randint(0, 16, (8, 4)) for _ in range(4)])
    tr.train(iterations=8)
    first = sum(l["score"] for l in tr.log[:4]) / 4
    last = sum(l["score"] for l in tr.log[-4:]) / 4
    assert last > first, (first, last)
    assert all(not p.requires_grad for p in eng.models["ref_model"].parameters())
