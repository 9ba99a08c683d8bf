"""``BF16Optimizer``: fp32 master copies for a model held entirely in bf16 (the ``half="bf16"`` case
without a sharded engine). The inner optimizer steps the fp32 masters; results are copied back.

State dict: ``{"optimizer_state_dict": ..., "fp32_from_fp16": [[tensor, ...] per group]}``.
(Reference: atorch/optimizers/bf16_optimizer.py:51-272.)
"""
from __future__ import annotations

import torch


class BF16Optimizer:
    def __init__(self, optimizer: torch.optim.Optimizer, grad_accumulate_in_fp32: bool = True):
        self.optimizer = optimizer
        self.pairs = []          # (low-precision param, fp32 master)
        for group in optimizer.param_groups:
            new = []
            for p in group["params"]:
                if p.dtype in (torch.bfloat16, torch.float16):
                    master = torch.nn.Parameter(p.detach().float().clone(), requires_grad=p.requires_grad)
                    if p in optimizer.state:
                        optimizer.state[master] = optimizer.state.pop(p)
                    self.pairs.append((p, master))
                    new.append(master)
                else:
                    new.append(p)
            group["params"] = new
        self.found_inf = False

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def state(self):
        return self.optimizer.state

    def zero_grad(self, set_to_none: bool = True):
        for p, m in self.pairs:
            p.grad = None
            m.grad = None
        self.optimizer.zero_grad(set_to_none=set_to_none)

    def _copy_grads(self):
        for p, m in self.pairs:
            if p.grad is not None:
                m.grad = p.grad.float() if m.grad is None else m.grad.add_(p.grad.float())
                p.grad = None

    def clip_grad_norm(self, max_norm: float, norm_type: float = 2.0):
        self._copy_grads()
        params = [q for g in self.optimizer.param_groups for q in g["params"] if q.grad is not None]
        return torch.nn.utils.clip_grad_norm_(params, max_norm, norm_type)

    @torch.no_grad()
    def step(self, closure=None):
        self._copy_grads()
        r = self.optimizer.step(closure) if closure is not None else self.optimizer.step()
        for p, m in self.pairs:
            p.copy_(m)
        return r

    def state_dict(self):
        groups, it = [], iter(self.pairs)
        masters = {id(m): m for _, m in self.pairs}
        for g in self.optimizer.param_groups:
            groups.append([q.detach().clone() for q in g["params"] if id(q) in masters])
        return {"optimizer_state_dict": self.optimizer.state_dict(), "fp32_from_fp16": groups}

    def load_state_dict(self, sd):
        self.optimizer.load_state_dict(sd["optimizer_state_dict"])
        masters = {id(m) for _, m in self.pairs}
        for g, saved in zip(self.optimizer.param_groups, sd["fp32_from_fp16"]):
            cur = [q for q in g["params"] if id(q) in masters]
            for q, s in zip(cur, saved):
                q.data.copy_(s)
        for p, m in self.pairs:
            p.data.copy_(m.data)
