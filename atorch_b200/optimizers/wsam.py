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
        """Average the gradients over the default process group: one all-reduce per dtype over a flattened
        copy instead of one per parameter."""
        if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1) or not params:
            return
        world = dist.get_world_size()
        by_dtype = {}
        for p in params:
            by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
        for grads in by_dtype.values():
            flat = torch._utils._flatten_dense_tensors(grads)
            flat.div_(world)
            dist.all_reduce(flat)
            torch._foreach_copy_(grads, torch._utils._unflatten_dense_tensors(flat, grads))

    def _grad_norm(self) -> torch.Tensor:
        dev = self.param_groups[0]["params"][0].device
        norms = []
        for g in self.param_groups:
            ps = self._with_grad(g)
            if not ps:
                continue
            grads = [p.grad for p in ps]
            ts = torch._foreach_mul(torch._foreach_abs(ps), grads) if g["adaptive"] else grads
            norms += [n.to(dev, torch.float32) for n in torch._foreach_norm(ts)]
        return torch.linalg.vector_norm(torch.stack(norms)) if norms else torch.zeros((), device=dev)

    @torch.no_grad()
    def first_step(self, zero_grad: bool = False) -> None:
        gnorm = self._grad_norm()
        for group in self.param_groups:
            ps = self._with_grad(group)
            if not ps:
                continue
            scale = (group["rho"] / (gnorm + group["sam_eps"])).item()
            e_ws = torch._foreach_mul([p.grad for p in ps], scale)
            if group["adaptive"]:
                torch._foreach_mul_(e_ws, torch._foreach_mul(ps, ps))
            torch._foreach_add_(ps, e_ws)
            for p, e in zip(ps, e_ws):
                self.state[p]["e_w"] = e
            self._avg_grads(ps)
        if self.max_norm is not None:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_norm)
        for group in self.param_groups:
            ps = self._with_grad(group)
            for p, g in zip(ps, torch._foreach_add([p.grad for p in ps], 0.0) if ps else []):
                self.state[p]["grad"] = g
        if zero_grad:
            self.zero_grad()

    @torch.no_grad()
    def second_step(self, zero_grad: bool = False) -> None:
        for group in self.param_groups:
            ps = self._with_grad(group)
            if not ps:
                continue
            self._avg_grads(ps)
            torch._foreach_sub_(ps, [self.state[p]["e_w"] for p in ps])
        if self.max_norm is not None:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_norm)
        for group in self.param_groups:
            ps = self._with_grad(group)
            if not ps:
                continue
            grads, first = [p.grad for p in ps], [self.state[p]["grad"] for p in ps]
            if not self.decouple:
                torch._foreach_mul_(grads, group["alpha"])
                torch._foreach_add_(grads, first, alpha=1.0 - group["alpha"])
            else:
                for p, sh in zip(ps, torch._foreach_sub(grads, first)):
                    self.state[p]["sharpness"] = sh
                torch._foreach_copy_(grads, first)
        self.base_optimizer.step()
        if self.decouple:
            for group in self.param_groups:
                ps = self._with_grad(group)
                if ps:
                    torch._foreach_add_(ps, [self.state[p]["sharpness"] for p in ps],
                                        alpha=-group["lr"] * group["alpha"])
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
