"""RMSNorm / LayerNorm with the sm_100a row kernels (fused residual add, deterministic dw).

Reference counterparts: ``AtorchRmsNorm`` (atorch/modules/transformer/rmsnorm.py:12) on the Triton
kernels of atorch/kernels/triton_jit/rmsnorm_kernel.py, and ``AtorchLayerNorm``
(atorch/modules/normalization/layernorm.py:7).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib


def rms_norm_reference(x, weight, eps=1e-6, residual=None):
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * weight.float()).to(x.dtype)
    return (y, x) if residual is not None else y


def layer_norm_reference(x, weight, bias, eps=1e-5):
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), weight.float(),
                                          None if bias is None else bias.float(), eps).to(x.dtype)


def _fwd(x2, res2, w, b, eps, ln):
    M, N = x2.shape
    y = torch.empty_like(x2)
    s = torch.empty_like(x2) if res2 is not None else None
    rstd = torch.empty(M, dtype=torch.float32, device=x2.device)
    mean = torch.empty(M, dtype=torch.float32, device=x2.device) if ln else None
    rc = _lib.lib().atb_norm_fwd(_lib.ptr(x2), _lib.ptr(res2), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), _lib.ptr(s),
                                 _lib.ptr(mean), _lib.ptr(rstd), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_float(eps),
                                 ctypes.c_int(int(ln)), ctypes.c_int(_lib.DT[x2.dtype]), _lib.stream_ptr())
    _lib.check(rc, "atb_norm_fwd")
    return y, s, mean, rstd


def _bwd(dy2, x2, w, mean, rstd, dres2, ln, need_db):
    M, N = x2.shape
    L = _lib.lib()
    parts = L.atb_norm_bwd_parts(ctypes.c_int(M))
    pdw = torch.empty(parts, N, dtype=torch.float32, device=x2.device)
    pdb = torch.empty(parts, N, dtype=torch.float32, device=x2.device) if (ln and need_db) else None
    dx = torch.empty_like(x2)
    rc = L.atb_norm_bwd(_lib.ptr(dy2), _lib.ptr(x2), _lib.ptr(w), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(dres2),
                        _lib.ptr(dx), _lib.ptr(pdw), _lib.ptr(pdb), ctypes.c_int(parts), ctypes.c_int(M),
                        ctypes.c_int(N), ctypes.c_int(int(ln)), ctypes.c_int(_lib.DT[x2.dtype]), _lib.stream_ptr())
    _lib.check(rc, "atb_norm_bwd")
    return dx, pdw, pdb, parts


def _colsum(partial, parts, out, accumulate):
    N = partial.shape[1]
    rc = _lib.lib().atb_colsum(_lib.ptr(partial), _lib.ptr(out), ctypes.c_int(parts), ctypes.c_int(N),
                               ctypes.c_int(_lib.DT[out.dtype]), ctypes.c_int(int(accumulate)), _lib.stream_ptr())
    _lib.check(rc, "atb_colsum")


def _param_grad(param, partial, parts):
    """Reduce the partial rows into ``param.main_grad`` (accumulating) or into a fresh grad tensor."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        first = getattr(param, "_atb_first", False)
        _colsum(partial, parts, mg, not first)
        param._atb_first = False
        param.grad_added_to_main_grad = True
        return None
    g = torch.empty_like(param)
    _colsum(partial, parts, g, False)
    return g


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, bias, eps, ln, carry=False):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, shp[-1])
            res2 = res2 if res2.is_contiguous() else res2.contiguous()
        y, s, mean, rstd = _fwd(x2, res2, weight, bias, eps, ln)
        ctx.save_for_backward(s if s is not None else x2, weight, mean, rstd)
        ctx.ln, ctx.shp, ctx.has_res = ln, shp, residual is not None
        ctx.w_ref, ctx.b_ref = weight, bias
        if residual is not None:
            return y.view(shp), s.view(shp)
        if carry:
            # second output: x itself (a second tensor over the same storage, no copy) for the residual path, so
            # that the gradient arriving through it is added inside the backward kernel
            return y.view(shp), torch.empty(0, dtype=x.dtype, device=x.device).set_(
                x.untyped_storage(), x.storage_offset(), x.shape, x.stride())
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy, dsum=None):
        xin, weight, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        d2 = None
        if dsum is not None:
            d2 = dsum.reshape(-1, dsum.shape[-1])
            d2 = d2 if d2.is_contiguous() else d2.contiguous()
        need_db = ctx.ln and ctx.b_ref is not None
        dx, pdw, pdb, parts = _bwd(dy2, xin, weight, mean, rstd, d2, ctx.ln, need_db)
        dw = _param_grad(ctx.w_ref, pdw, parts) if ctx.needs_input_grad[2] else None
        db = _param_grad(ctx.b_ref, pdb, parts) if (need_db and ctx.needs_input_grad[3]) else None
        dx = dx.view(ctx.shp)
        return dx, (dx if ctx.has_res else None), dw, db, None, None, None


def _kernel_ok(x, weight):
    return (_lib.use_kernels(x, weight) and x.dtype in _lib.DT and weight.dtype == x.dtype
            and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
             residual: Optional[torch.Tensor] = None, carry: bool = False):
    """``y = rmsnorm(x [+ residual]) * weight``; with ``residual`` also returns the sum ``x + residual``.

    ``carry`` (without ``residual``): also return ``x`` for the residual branch of a pre-norm block. Using that
    second output instead of ``x`` itself makes both gradients of ``x`` (through the norm and through the
    residual path) arrive in one backward call, whose kernel adds them, instead of autograd summing them with a
    separate pass over the activations."""
    if not _kernel_ok(x, weight):
        y = rms_norm_reference(x, weight, eps, residual)
        return (y, x) if (carry and residual is None) else y
    if carry and residual is None:
        return _Norm.apply(x, None, weight, None, eps, False, True)
    return _Norm.apply(x, residual, weight, None, eps, False)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, eps: float = 1e-5):
    if not _kernel_ok(x, weight) or (bias is not None and bias.dtype != x.dtype):
        return layer_norm_reference(x, weight, bias, eps)
    return _Norm.apply(x, None, weight, bias, eps, True)
