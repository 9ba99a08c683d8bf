"""Fused flat-buffer optimizer steps (AdamW, AGD, Nesterov outer step) and the sum-of-squares
reduction used for gradient-norm clipping.

Reference counterparts: torch AdamW under FSDP, atorch/optimizers/agd.py:73-155,
torch.optim.SGD(nesterov) in atorch/local_sgd/DDP/outer_optim_model_averager.py:161-192.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from .. import _lib


def adamw_reference(master, m, v, grad, param_lp, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                    adamw_mode=True):
    g = grad.float() * grad_scale
    if adamw_mode:
        master.mul_(1.0 - lr * weight_decay)
    else:
        g = g + weight_decay * master
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    master.addcdiv_(m / bc1, denom, value=-lr)
    if param_lp is not None:
        param_lp.copy_(master)


def adamw_step(master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad: torch.Tensor,
               param_lp: Optional[torch.Tensor], lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, step: int, grad_scale: float = 1.0,
               grad_scale_tensor: Optional[torch.Tensor] = None, adamw_mode: bool = True,
               max_blocks: int = 0) -> None:
    """One fused AdamW step on flat fp32 ``master/m/v`` from a flat bf16/fp32 ``grad``; writes the
    bf16 working copy ``param_lp`` (may be None). ``grad_scale_tensor`` is an optional device scalar
    multiplied into the gradient (clipping coefficient computed on the device). ``max_blocks`` caps the grid
    (0 = enough CTAs to fill the GPU) for launches meant to share the SMs with other kernels."""
    n = master.numel()
    ok = (_lib.use_kernels(master, grad) and master.dtype == torch.float32 and grad.dtype in (torch.bfloat16, torch.float32)
          and (param_lp is None or param_lp.dtype == torch.bfloat16))
    if not ok:
        gs = grad_scale * (float(grad_scale_tensor) if grad_scale_tensor is not None else 1.0)
        return adamw_reference(master, m, v, grad, param_lp, lr, beta1, beta2, eps, weight_decay, step, gs, adamw_mode)
    rc = _lib.lib().atb_adamw(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(grad), _lib.ptr(param_lp),
                              ctypes.c_longlong(n), ctypes.c_float(lr), ctypes.c_float(beta1), ctypes.c_float(beta2),
                              ctypes.c_float(eps), ctypes.c_float(weight_decay), ctypes.c_int(step),
                              ctypes.c_float(grad_scale), _lib.ptr(grad_scale_tensor), ctypes.c_int(int(adamw_mode)),
                              ctypes.c_int(_lib.DT[grad.dtype]), ctypes.c_int(max_blocks), _lib.stream_ptr())
    _lib.check(rc, "atb_adamw")


def agd_reference(master, m, v, grad, param_lp, lr, beta1, beta2, delta, weight_decay, step, grad_scale=1.0,
                  clip=None, decouple=True, fixed_decay=False):
    g = grad.float() * grad_scale
    if decouple:
        master.mul_(1.0 - weight_decay if fixed_decay else 1.0 - lr * weight_decay)
    else:
        g = g + weight_decay * master
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    m_old = m.clone()
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    if step == 1:
        s = m / bc1
    else:
        s = m / bc1 - m_old / (1 - beta1 ** (step - 1))
    v.mul_(beta2).addcmul_(s, s, value=1 - beta2)
    den = torch.maximum(v.sqrt(), torch.full_like(v, delta * math.sqrt(bc2)))
    u = m / den
    if clip is not None and clip > 0:
        u = u.clamp(-clip, clip)
    master.add_(u, alpha=-lr * math.sqrt(bc2) / bc1)
    if param_lp is not None:
        param_lp.copy_(master)


def agd_step(master, m, v, grad, param_lp, lr, beta1, beta2, delta, weight_decay, step, grad_scale=1.0,
             grad_scale_tensor=None, clip=None, decouple=True, fixed_decay=False) -> None:
    """One fused AGD step (same buffer contract as :func:`adamw_step`)."""
    n = master.numel()
    ok = (_lib.use_kernels(master, grad) and master.dtype == torch.float32 and grad.dtype in (torch.bfloat16, torch.float32)
          and (param_lp is None or param_lp.dtype == torch.bfloat16))
    if not ok:
        gs = grad_scale * (float(grad_scale_tensor) if grad_scale_tensor is not None else 1.0)
        return agd_reference(master, m, v, grad, param_lp, lr, beta1, beta2, delta, weight_decay, step, gs, clip,
                             decouple, fixed_decay)
    rc = _lib.lib().atb_agd(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(grad), _lib.ptr(param_lp),
                            ctypes.c_longlong(n), ctypes.c_float(lr), ctypes.c_float(beta1), ctypes.c_float(beta2),
                            ctypes.c_float(delta), ctypes.c_float(weight_decay), ctypes.c_int(step),
                            ctypes.c_float(grad_scale), _lib.ptr(grad_scale_tensor),
                            ctypes.c_float(clip if clip else 0.0), ctypes.c_int(int(decouple)),
                            ctypes.c_int(int(fixed_decay)), ctypes.c_int(_lib.DT[grad.dtype]), _lib.stream_ptr())
    _lib.check(rc, "atb_agd")


def sum_squares(x: torch.Tensor) -> torch.Tensor:
    """fp32 scalar tensor: sum of squares of ``x`` (deterministic two-pass on the GPU)."""
    if not (_lib.use_kernels(x) and x.dtype in (torch.bfloat16, torch.float32) and x.is_contiguous()):
        return x.float().pow(2).sum()
    L = _lib.lib()
    parts = L.atb_sumsq_parts()
    partial = torch.empty(parts, dtype=torch.float32, device=x.device)
    rc = L.atb_sumsq(_lib.ptr(x), ctypes.c_longlong(x.numel()), _lib.ptr(partial), ctypes.c_int(_lib.DT[x.dtype]),
                     _lib.stream_ptr())
    _lib.check(rc, "atb_sumsq")
    return partial.sum()


def outer_sgd_reference(synced, buf, pseudo_grad, param, lr, momentum, nesterov, first_step, scale=1.0):
    g = pseudo_grad.float() * scale
    if first_step:
        buf.copy_(g)
    else:
        buf.mul_(momentum).add_(g)
    upd = g + momentum * buf if nesterov else buf
    synced.add_(upd, alpha=-lr)
    if param is not None:
        param.copy_(synced)


def outer_sgd_step(synced: torch.Tensor, buf: torch.Tensor, pseudo_grad: torch.Tensor,
                   param: Optional[torch.Tensor], lr: float, momentum: float, nesterov: bool, first_step: bool,
                   scale: float = 1.0) -> None:
    """Local-SGD outer step: momentum/Nesterov SGD on the last synchronised weights from a reduced
    pseudo-gradient, then write the result back into the live parameters (fp32 or bf16)."""
    ok = (_lib.use_kernels(synced, pseudo_grad) and synced.dtype == torch.float32 and pseudo_grad.dtype == torch.float32
          and (param is None or param.dtype in (torch.float32, torch.bfloat16)))
    if not ok:
        return outer_sgd_reference(synced, buf, pseudo_grad, param, lr, momentum, nesterov, first_step, scale)
    pf = param if (param is not None and param.dtype == torch.float32) else None
    pb = param if (param is not None and param.dtype == torch.bfloat16) else None
    rc = _lib.lib().atb_outer_sgd(_lib.ptr(synced), _lib.ptr(buf), _lib.ptr(pseudo_grad), _lib.ptr(pf), _lib.ptr(pb),
                                  ctypes.c_longlong(synced.numel()), ctypes.c_float(lr), ctypes.c_float(momentum),
                                  ctypes.c_int(int(nesterov)), ctypes.c_int(int(first_step)), ctypes.c_float(scale),
                                  _lib.stream_ptr())
    _lib.check(rc, "atb_outer_sgd")
