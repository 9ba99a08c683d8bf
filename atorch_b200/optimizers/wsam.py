"""Weighted sharpness-aware minimisation (WSAM): two forward/backward passes per step.

    pass 1 at w        : g = grad;  e = rho * g / (||g|| + eps)   (adaptive: e *= w^2, norm uses |w| g)
                         w += e; gradients averaged over the data-parallel group, g saved
    pass 2 at w + e    : g_s = grad (averaged);  w -= e
    combine (alpha = gamma / (1 - gamma)):
        coupled   : grad = alpha * g_s + (1 - alpha) * g, then the base optimizer steps
        decoupled : base optimizer steps with g, then w -= lr * alpha * (g_s - g)
The foreach forms below keep the work to a handful of fused tensor-list kernels per step.
(Reference: atorch/optimizers/wsam.py:11-138, BN helpers atorch/optimizers/utils.py:6-27.)
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.nn.modules.batchnorm import _BatchNorm


def disable_running_stats(model) -> None:
    def f(m):
        if isinstance(m, _BatchNorm):
            m.backup_momentum = m.momentum
            m.momentum = 0
    model.apply(f)


def enable_running_stats(model) -> None:
    def f(m):
        if isinstance(m, _BatchNorm) and hasattr(m, "backup_momentum"):
            m.momentum = m.backup_momentum
    model.apply(f)


class WeightedSAM(torch.optim.Optimizer):
    def __init__(self, model, base_optimizer, rho: float = 0.05, gamma: float = 0.9, sam_eps: float = 1e-12,
                 adaptive: bool = False, decouple: bool = True, max_norm=None, **kwargs):
        assert rho >= 0.0, f"Invalid rho, should be non-negative: {rho}"
        self.model, self.base_optimizer = model, base_optimizer
        self.decouple, self.max_norm = decouple, max_norm
        defaults = dict(rho=rho, alpha=gamma / (1 - gamma), sam_eps=sam_eps, adaptive=adaptive, **kwargs)
        defaults.update(base_optimizer.defaults)
        super().__init__(base_optimizer.param_groups, defaults)

    def _with_grad(self, group):
        return [p for p in group["params"] if p.grad is not None]

    def _avg_grads(self, params) -> None:
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            world = dist.get_world_size()
            for p in params:
                p.grad.div_(world)
                dist.all_reduce(p.grad)

    def _grad_norm(self) -> torch.Tensor:
        dev = self.param_groups[0]["params"][0].device
        norms = []
        for g in self.param_groups:
            for p in self._with_grad(g):
                t = (p.abs() * p.grad) if g["adaptive"] else p.grad
                norms.append(torch.linalg.vector_norm(t.float()).to(dev))
        return torch.linalg.vector_norm(torch.stack(norms)) if norms else torch.zeros((), device=dev)

    @torch.no_grad()
    def first_step(self, zero_grad: bool = False) -> None:
        gnorm = self._grad_norm()
        for group in self.param_groups:
            scale = group["rho"] / (gnorm + group["sam_eps"])
            ps = self._with_grad(group)
            for p in ps:
                e_w = (p.pow(2) if group["adaptive"] else 1.0) * p.grad * scale.to(p)
                p.add_(e_w)
                self.state[p]["e_w"] = e_w
            self._avg_grads(ps)
        if self.max_norm is not None:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_norm)
        for group in self.param_groups:
            for p in self._with_grad(group):
                self.state[p]["grad"] = p.grad.detach().clone()
        if zero_grad:
            self.zero_grad()

    @torch.no_grad()
    def second_step(self, zero_grad: bool = False) -> None:
        for group in self.param_groups:
            ps = self._with_grad(group)
            self._avg_grads(ps)
            for p in ps:
                p.sub_(self.state[p]["e_w"])
        if self.max_norm is not None:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_norm)
        for group in self.param_groups:
            for p in self._with_grad(group):
                st = self.state[p]
                if not self.decouple:
                    p.grad.mul_(group["alpha"]).add_(st["grad"], alpha=1.0 - group["alpha"])
                else:
                    st["sharpness"] = p.grad.detach() - st["grad"]
                    p.grad.copy_(st["grad"])
        self.base_optimizer.step()
        if self.decouple:
            for group in self.param_groups:
                for p in self._with_grad(group):
                    p.add_(self.state[p]["sharpness"], alpha=-group["lr"] * group["alpha"])
        if zero_grad:
            self.zero_grad()

    @torch.no_grad()
    def step(self, closure=None):
        assert closure is not None, "Sharpness Aware Minimization requires closure, but it was not provided"
        closure = torch.enable_grad()(closure)
        enable_running_stats(self.model)
        loss = closure()
        self.first_step(zero_grad=True)
        disable_running_stats(self.model)
        closure()
        self.second_step()
        return loss
