"""Low-bit optimizers: first/second moments stored as 4- or 8-bit codes with one fp32 absmax per
group of 128 (4-bit) or 2048 (8-bit) elements, de-quantised, updated and re-quantised each step.
Signed states (first moment) use a signed code book, non-negative ones (second moment) an unsigned
one; tensors below ``min_quant_size`` (4096) elements stay in fp32.

``Q_AdamW``, ``Q_AGD`` (AGD's momentum-difference preconditioner), ``Q_CAME`` and ``Q_Adafactor``
(factored second moments; the factors are small and stay fp32, the momentum is quantised).
(Reference: atorch/optimizers/low_bit/{optim.py,functional.py,config.py}.)
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch.optim import Optimizer

from ...ops import lowbit


class _QState:
    """One quantised state tensor."""

    def __init__(self, like: torch.Tensor, bits: int, signed: bool, group_size: int, min_quant_size: int,
                 stochastic: bool):
        self.shape, self.n, self.device = like.shape, like.numel(), like.device
        self.bits, self.signed, self.group_size, self.stochastic = bits, signed, group_size, stochastic
        self.quantised = self.n >= min_quant_size and bits < 32
        self.qmap = lowbit.create_dynamic_map(signed, bits).to(like.device) if self.quantised else None
        self.code = self.absmax = None
        self.full = None if self.quantised else torch.zeros_like(like, dtype=torch.float32)
        self.step = 0

    def get(self) -> torch.Tensor:
        if not self.quantised:
            return self.full
        if self.code is None:
            return torch.zeros(self.shape, dtype=torch.float32, device=self.device)
        return lowbit.unpack_nonlinear(self.code, self.absmax, self.qmap, self.n, self.bits, self.group_size).view(self.shape)

    def set(self, value: torch.Tensor) -> None:
        if not self.quantised:
            self.full = value
            return
        self.step += 1
        self.code, self.absmax = lowbit.pack_nonlinear(value, self.qmap, self.bits, self.group_size, self.stochastic,
                                                       seed=self.step)

    def state_dict(self):
        return {"code": self.code, "absmax": self.absmax, "full": self.full, "step": self.step}

    def load_state_dict(self, sd):
        self.code, self.absmax, self.full, self.step = sd["code"], sd["absmax"], sd["full"], sd["step"]


class _LowBitBase(Optimizer):
    def __init__(self, params, defaults, q_bits: int = 4, min_quant_size: int = 4096, stochastic_rounding: bool = False):
        defaults = dict(defaults, q_bits=q_bits)
        super().__init__(params, defaults)
        self.q_bits, self.min_quant_size, self.stochastic = q_bits, min_quant_size, stochastic_rounding
        self.group_size = 128 if q_bits <= 4 else 2048

    def _qstate(self, p, signed: bool) -> _QState:
        return _QState(p, self.q_bits, signed, self.group_size, self.min_quant_size, self.stochastic)


class Q_AdamW(_LowBitBase):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, q_bits=4,
                 min_quant_size=4096, stochastic_rounding=False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay), q_bits, min_quant_size,
                         stochastic_rounding)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"], st["m"], st["v"] = 0, self._qstate(p, True), self._qstate(p, False)
                st["step"] += 1
                t = st["step"]
                grad = p.grad.float()
                m = st["m"].get().mul_(b1).add_(grad, alpha=1 - b1)
                v = st["v"].get().mul_(b2).addcmul_(grad, grad, value=1 - b2)
                p.mul_(1 - g["lr"] * g["weight_decay"])
                denom = (v / (1 - b2 ** t)).sqrt_().add_(g["eps"])
                p.addcdiv_((m / (1 - b1 ** t)).to(p.dtype), denom.to(p.dtype), value=-g["lr"])
                st["m"].set(m)
                st["v"].set(v)
        return loss


class Q_AGD(_LowBitBase):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), delta=1e-5, weight_decay=0.0, clip=None, q_bits=4,
                 min_quant_size=4096, stochastic_rounding=False):
        super().__init__(params, dict(lr=lr, betas=betas, delta=delta, weight_decay=weight_decay, clip=clip), q_bits,
                         min_quant_size, stochastic_rounding)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"], st["m"], st["v"] = 0, self._qstate(p, True), self._qstate(p, False)
                st["step"] += 1
                t = st["step"]
                grad = p.grad.float()
                p.mul_(1 - g["lr"] * g["weight_decay"])
                m_old = st["m"].get()
                m = m_old.mul(b1).add_(grad, alpha=1 - b1)
                bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
                s = m / bc1 if t == 1 else m / bc1 - m_old / (1 - b1 ** (t - 1))
                v = st["v"].get().mul_(b2).addcmul_(s, s, value=1 - b2)
                den = v.sqrt().clamp_(min=g["delta"] * math.sqrt(bc2))
                u = m / den
                if g["clip"] is not None:
                    u.clamp_(-g["clip"], g["clip"])
                p.add_(u.to(p.dtype), alpha=-g["lr"] * math.sqrt(bc2) / bc1)
                st["m"].set(m)
                st["v"].set(v)
        return loss


def _rms(t):
    return t.norm(2) / (t.numel() ** 0.5)


class Q_Adafactor(_LowBitBase):
    """Adafactor with factored second moments (row/column means) for matrices and quantised momentum."""

    def __init__(self, params, lr=1e-3, eps=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=-0.8, beta1=0.9,
                 weight_decay=0.0, q_bits=4, min_quant_size=4096, stochastic_rounding=False):
        super().__init__(params, dict(lr=lr, eps=eps, clip_threshold=clip_threshold, decay_rate=decay_rate,
                                      beta1=beta1, weight_decay=weight_decay), q_bits, min_quant_size,
                         stochastic_rounding)

    def _second_moment_update(self, st, grad, g, beta2t):
        sq = grad * grad + g["eps"][0]
        if grad.dim() >= 2:
            r, c = st["row"], st["col"]
            r.mul_(beta2t).add_(sq.mean(-1), alpha=1 - beta2t)
            c.mul_(beta2t).add_(sq.mean(-2), alpha=1 - beta2t)
            rf = (r / r.mean(-1, keepdim=True)).rsqrt_().unsqueeze(-1)
            cf = c.unsqueeze(-2).rsqrt()
            return rf * cf * grad
        v = st["v"]
        v.mul_(beta2t).add_(sq, alpha=1 - beta2t)
        return grad * v.rsqrt()

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                grad = p.grad.float()
                if not st:
                    st["step"] = 0
                    if grad.dim() >= 2:
                        st["row"] = torch.zeros(grad.shape[:-1], device=p.device)
                        st["col"] = torch.zeros(grad.shape[:-2] + grad.shape[-1:], device=p.device)
                    else:
                        st["v"] = torch.zeros_like(grad)
                    if g["beta1"]:
                        st["m"] = self._qstate(p, True)
                st["step"] += 1
                beta2t = 1.0 - st["step"] ** g["decay_rate"]
                u = self._second_moment_update(st, grad, g, beta2t)
                u.div_((_rms(u) / g["clip_threshold"]).clamp_(min=1.0))
                if g["beta1"]:
                    m = st["m"].get().mul_(g["beta1"]).add_(u, alpha=1 - g["beta1"])
                    st["m"].set(m)
                    u = m
                p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(u.to(p.dtype), alpha=-g["lr"])
        return loss


class Q_CAME(Q_Adafactor):
    """CAME: Adafactor-style update whose confidence (squared deviation of the update from its momentum)
    is itself factored and used to rescale the step."""

    def __init__(self, params, lr=2e-4, eps=(1e-30, 1e-16), clip_threshold=1.0, betas=(0.9, 0.999, 0.9999),
                 weight_decay=0.0, q_bits=4, min_quant_size=4096, stochastic_rounding=False):
        _LowBitBase.__init__(self, params, dict(lr=lr, eps=eps, clip_threshold=clip_threshold, betas=betas,
                                                weight_decay=weight_decay, beta1=betas[0]), q_bits, min_quant_size,
                             stochastic_rounding)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2, b3 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                grad = p.grad.float()
                if not st:
                    st["step"] = 0
                    if grad.dim() >= 2:
                        st["row"] = torch.zeros(grad.shape[:-1], device=p.device)
                        st["col"] = torch.zeros(grad.shape[:-2] + grad.shape[-1:], device=p.device)
                        st["res_row"], st["res_col"] = torch.zeros_like(st["row"]), torch.zeros_like(st["col"])
                    else:
                        st["v"] = torch.zeros_like(grad)
                    st["m"] = self._qstate(p, True)
                st["step"] += 1
                u = self._second_moment_update(st, grad, g, b2)
                u.div_((_rms(u) / g["clip_threshold"]).clamp_(min=1.0))
                m = st["m"].get().mul_(b1).add_(u, alpha=1 - b1)
                st["m"].set(m)
                if grad.dim() >= 2:
                    res = (u - m) ** 2 + g["eps"][1]
                    rr, rc = st["res_row"], st["res_col"]
                    rr.mul_(b3).add_(res.mean(-1), alpha=1 - b3)
                    rc.mul_(b3).add_(res.mean(-2), alpha=1 - b3)
                    rf = (rr / rr.mean(-1, keepdim=True)).rsqrt_().unsqueeze(-1)
                    upd = rf * rc.unsqueeze(-2).rsqrt() * m
                else:
                    upd = m
                p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(upd.to(p.dtype), alpha=-g["lr"])
        return loss
