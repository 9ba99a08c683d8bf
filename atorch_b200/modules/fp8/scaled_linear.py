"""``ScaledLinear``: ``nn.Linear`` whose three GEMMs (fprop, dgrad, wgrad) run in block-scaled fp8.

tileblock recipe (the one the MoE benchmark names): input and gradient e4m3 with 1x128 scales,
weight e4m3 with 128x128 scales, fp32 accumulation:

    fprop  y  = Q_tile(x)   . Q_block(W)^T
    dgrad  dx = Q_tile(dy)  . Q_block(W^T)^T            (transposed weight copy from the same kernel)
    wgrad  dW = Q_tile(dy^T). Q_tile(x^T)^T             (both quantised along the token dim)

Quantised weights are cached until the weight changes (version counter), so micro-batches of one
step reuse them. Shapes that do not fit the block sizes fall back to the bf16 GEMM, like the
reference. ``scale_method`` "tensorwise" / "axiswise" use per-tensor / per-row scales through the
same kernels (a constant scale map).
(Reference: atorch/modules/fp8/scaled_linear.py:19-532.)
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ... import ops
from . import quantize as Q


def fp8_shapes_ok(in_features: int, out_features: int, block: int = 128) -> bool:
    return in_features % block == 0 and out_features % block == 0


class _WeightCache:
    def __init__(self):
        self.version = None
        self.q = self.s = self.qt = None

    def get(self, w: torch.Tensor, pow2: bool):
        v = (w._version, w.data_ptr())
        if self.version != v:
            self.q, self.s, self.qt = Q.block_quantize(w.detach(), with_transpose=True, pow2=pow2)
            self.version = v
        return self.q, self.s, self.qt


class _ScaledLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, cache: _WeightCache, pow2: bool):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        wq, ws, wqt = cache.get(weight, pow2)
        xq, xs = Q.tile_quantize(x2, pow2)
        y = Q.scaled_gemm(xq, xs, wq, ws, b_row_mode=False, out_dtype=x.dtype)
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.save_for_backward(x2, weight)
        ctx.cache, ctx.pow2, ctx.shp, ctx.has_bias = cache, pow2, shp, bias is not None
        ctx.w_ref = weight
        return y.view(*shp[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        wq, ws, wqt = ctx.cache.get(weight, ctx.pow2)
        dx = dw = db = None
        M = dy2.shape[0]
        if ctx.needs_input_grad[0]:
            gq, gs = Q.tile_quantize(dy2, ctx.pow2)
            dx = Q.scaled_gemm(gq, gs, wqt, ws.t().contiguous(), b_row_mode=False, out_dtype=x2.dtype).view(ctx.shp)
        if ctx.needs_input_grad[1]:
            if M % 128 == 0:
                gqt, gst = Q.tile_quantize_transposed(dy2, ctx.pow2)     # [N, M]
                xqt, xst = Q.tile_quantize_transposed(x2, ctx.pow2)      # [K, M]
                mg = getattr(ctx.w_ref, "main_grad", None)
                if mg is not None and mg.dtype == torch.float32:
                    Q.scaled_gemm(gqt, gst, xqt, xst, b_row_mode=True, out=mg, accumulate=True)
                    ctx.w_ref.grad_added_to_main_grad = True
                else:
                    dw = Q.scaled_gemm(gqt, gst, xqt, xst, b_row_mode=True, out_dtype=weight.dtype)
            else:
                dw = ops.gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db, None, None


class ScaledLinear(nn.Linear):
    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None, scale_method="tileblock",
                 scale_block_size: int = 128, quantization_method="default", compute_method="default",
                 pow2_scale: bool = False):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        assert scale_block_size == 128, "this build implements 128-wide scale blocks"
        self.scale_method, self.pow2_scale = scale_method, pow2_scale
        self.quantization_method, self.compute_method = quantization_method, compute_method
        self.use_fp8 = True
        self._cache = _WeightCache()

    @classmethod
    def from_linear(cls, lin: nn.Linear, **kw) -> "ScaledLinear":
        m = cls(lin.in_features, lin.out_features, bias=lin.bias is not None, device=lin.weight.device,
                dtype=lin.weight.dtype, **kw)
        m.weight = lin.weight
        if lin.bias is not None:
            m.bias = lin.bias
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ok = self.use_fp8 and fp8_shapes_ok(self.in_features, self.out_features) and x.dtype == torch.bfloat16
        if not ok:
            return ops.linear(x, self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype), self.bias)
        w = self.weight if self.weight.dtype == torch.bfloat16 else self.weight.to(torch.bfloat16)
        if w is not self.weight:       # derived copy: cache keyed on the parameter's own version
            w._version_src = self.weight
        return _ScaledLinearFn.apply(x, w, self.bias, self._cache, self.pow2_scale)
