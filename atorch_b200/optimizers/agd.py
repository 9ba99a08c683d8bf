"""AGD: optimizer that preconditions with the *difference of successive bias-corrected momenta*
and switches to SGD-with-momentum behaviour where that difference is small.

Per parameter and step t (g = gradient, after optional coupled weight decay):
    m_t = b1 m_{t-1} + (1-b1) g
    s_t = m_t/(1-b1^t) - m_{t-1}/(1-b1^{t-1})        (t = 1: m_1/(1-b1))
    v_t = b2 v_{t-1} + (1-b2) s_t^2                   (amsgrad: running max of v)
    den = max(sqrt(v_t), delta * sqrt(1-b2^t))
    u   = m_t / den  (optionally clamped to [-clip, clip])
    p  -= lr * sqrt(1-b2^t)/(1-b1^t) * u
Decoupled weight decay multiplies p by (1 - lr*wd) (or (1 - wd) with ``fixed_decay``) first. The
``win`` variant (no separate weight decay) keeps a conservative sequence z, zero at the start (z -= step*u,
shrunk by 1/(1+wd*step)) and sets
p = tau*p - tau*2*step*u + 2*tau*z with tau = 1/(3 + 2*step*wd).

The update runs through the fused flat kernel (csrc/optim.cu) for CUDA fp32 parameters without
amsgrad/win; otherwise through the PyTorch expressions below.
(Reference: atorch/optimizers/agd.py:18-155, docs/README-AGD.md.)
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch.optim import Optimizer

from .. import ops


class AGD(Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), delta: float = 1e-5, weight_decay: float = 0.0,
                 weight_decouple: bool = True, fixed_decay: bool = False, amsgrad: bool = False, win: bool = False,
                 clip: Optional[float] = None):
        if lr < 0 or delta < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1:
            raise ValueError("invalid AGD hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, delta=delta, weight_decay=weight_decay,
                                      weight_decouple=weight_decouple, fixed_decay=fixed_decay, amsgrad=amsgrad,
                                      win=win, clip=clip))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("AGD does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    if group["amsgrad"]:
                        st["max_exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    if group["win"]:
                        st["z"] = torch.zeros_like(p, memory_format=torch.preserve_format)   # as the reference does
                st["step"] += 1
                t = st["step"]
                fused = (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and not group["amsgrad"]
                         and not group["win"] and p.grad.is_contiguous())
                if fused:
                    ops.agd_step(p.data.view(-1), st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1),
                                 p.grad.view(-1), None, group["lr"], b1, b2, group["delta"], group["weight_decay"],
                                 t, clip=group["clip"], decouple=group["weight_decouple"],
                                 fixed_decay=group["fixed_decay"])
                    continue
                self._reference_update(p, p.grad, st, group, t)
        return loss

    @staticmethod
    def _reference_update(p, grad, st, group, t):
        b1, b2 = group["betas"]
        lr, wd = group["lr"], group["weight_decay"]
        m, v = st["exp_avg"], st["exp_avg_sq"]
        bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
        if not group["win"]:              # with win the decay lives in the z / tau expressions below
            if group["weight_decouple"]:
                p.mul_(1 - wd if group["fixed_decay"] else 1 - lr * wd)
            elif wd != 0:
                grad = grad.add(p, alpha=wd)
        m_old = m.clone()
        m.mul_(b1).add_(grad, alpha=1 - b1)
        s = m / bc1 if t == 1 else m / bc1 - m_old / (1 - b1 ** (t - 1))
        v.mul_(b2).addcmul_(s, s, value=1 - b2)
        if group["amsgrad"]:
            torch.maximum(st["max_exp_avg_sq"], v, out=st["max_exp_avg_sq"])
            root = st["max_exp_avg_sq"].sqrt()
        else:
            root = v.sqrt()
        den = torch.clamp(root, min=group["delta"] * math.sqrt(bc2))
        u = m / den
        if group["clip"] is not None:
            u.clamp_(-group["clip"], group["clip"])
        step = lr * math.sqrt(bc2) / bc1
        if group["win"]:
            # Win acceleration: a conservative sequence z and a reckless step of twice the size,
            # mixed 1/3 : 2/3. z starts at zero and the ordinary weight decay is skipped, both as in the reference,
            # whose trajectory tests/test_reference_parity_cpu.py reproduces
            z = st["z"]
            z.add_(u, alpha=-step).mul_(1.0 / (1.0 + wd * step))
            step2 = 2.0 * step
            tau = 1.0 / (3.0 + step2 * wd)
            p.mul_(tau).add_(u, alpha=-tau * step2).add_(z, alpha=2.0 * tau)
        else:
            p.add_(u, alpha=-step)
