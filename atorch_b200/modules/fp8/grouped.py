"""Grouped block-scaled fp8 linear: consecutive row groups times one weight per group.

``grouped_scaled_linear(x, w, sizes)`` computes ``y[g] = x[g] W[g]^T`` (``w`` is ``[G, N, K]``) with the
fprop / dgrad / wgrad recipes of :mod:`scaled_linear`. Activations are quantised ONCE for all groups
(row strips do not cross groups along K), weights per group with a per-group cache.
(Reference: ``ATorchGroupedLinear`` in atorch/modules/fp8/quantized_grouped_linear.py:36-584, which
depends on the closed ``kitchen`` package.)
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from ... import ops
from . import quantize as Q


class _GroupedScaledFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, sizes: Tuple[int, ...], pow2: bool):
        G, N, K = w.shape
        xq, xs = Q.tile_quantize(x, pow2)
        out = torch.empty(x.shape[0], N, dtype=x.dtype, device=x.device)
        wq = [Q.block_quantize(w[g].detach(), with_transpose=True, pow2=pow2) for g in range(G)]
        r = 0
        for g, n in enumerate(sizes):
            if n:
                Q.scaled_gemm(xq[r: r + n], xs[r: r + n], wq[g][0], wq[g][1], out=out[r: r + n])
            r += n
        ctx.save_for_backward(x, w)
        ctx.sizes, ctx.pow2, ctx.wq = sizes, pow2, wq
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        gq, gs = Q.tile_quantize(dy, ctx.pow2)
        dx = torch.empty_like(x)
        dw = torch.zeros_like(w)
        r = 0
        for g, n in enumerate(ctx.sizes):
            if n:
                q, s, qt = ctx.wq[g]
                Q.scaled_gemm(gq[r: r + n], gs[r: r + n], qt, s.t().contiguous(), out=dx[r: r + n])
                if n % 128 == 0:
                    a, a_s = Q.tile_quantize_transposed(dy[r: r + n], ctx.pow2)
                    b, b_s = Q.tile_quantize_transposed(x[r: r + n], ctx.pow2)
                    Q.scaled_gemm(a, a_s, b, b_s, b_row_mode=True, out=dw[g])
                else:   # ragged group: the token dim cannot be cut into 128-strips
                    ops.gemm(dy[r: r + n], x[r: r + n], a_mn=True, b_mn=True, out=dw[g])
            r += n
        return dx, dw, None, None


def grouped_scaled_linear(x: torch.Tensor, w: torch.Tensor, sizes: Sequence[int], pow2: bool = False) -> torch.Tensor:
    G, N, K = w.shape
    if x.dtype != torch.bfloat16 or K % 128 or N % 128:
        return ops.moe.grouped_gemm(x, w.contiguous(), list(sizes), trans_b=True) if hasattr(ops, "moe") else \
            torch.cat([x[sum(sizes[:g]): sum(sizes[:g + 1])] @ w[g].t() for g in range(G)])
    wc = w if w.is_contiguous() else w.contiguous()
    return _GroupedScaledFn.apply(x, wc.to(torch.bfloat16) if wc.dtype != torch.bfloat16 else wc,
                                  tuple(int(s) for s in sizes), pow2)
