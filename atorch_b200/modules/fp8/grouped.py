"""Grouped block-scaled fp8 linear: consecutive row groups times one weight per group.

``grouped_scaled_linear(x, weights, sizes)`` computes ``y[g] = x[g] W[g]^T`` (each ``W[g]`` is ``[N, K]``;
``weights`` is a list of such tensors or one ``[G, N, K]`` tensor) with the fprop / dgrad / wgrad recipes of
:mod:`scaled_linear`. Activations are quantised ONCE for all groups (row strips do not cross groups along K).

Weights are quantised through a ``WeightQuantCache``: one entry per group holding the e4m3 weight, its
128x128 scales and the transposed copy for dgrad. An entry is refreshed when the weight changed (version
counter / storage) or when the caller asks for it - ``ATorchGroupedLinear`` does so on the first micro-batch
of a step and reuses the entries for the later ones. Weight gradients go into ``weight.main_grad`` when the
parameter has one and ``fuse_wgrad_accumulation`` is set.
(Reference: ``ATorchGroupedLinear`` in atorch/modules/fp8/quantized_grouped_linear.py:36-584 with its
``QuantizeResultCache``, which depends on the closed ``kitchen`` package.)
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple, Union

import torch

from ... import ops
from . import quantize as Q


class WeightQuantCache:
    """Quantised weights of the groups of one grouped linear."""

    def __init__(self):
        self.entries: List[Optional[tuple]] = []
        self.keys: List[Optional[tuple]] = []
        self.hits = self.misses = 0

    def get(self, g: int, w: torch.Tensor, pow2: bool, refresh: bool, origin: Optional[torch.Tensor] = None):
        """``w``: the contiguous weight to quantise; ``origin``: the tensor whose identity (storage, view
        geometry, version counter) stands for its values - the parameter view ``w`` was copied from."""
        while len(self.entries) <= g:
            self.entries.append(None)
            self.keys.append(None)
        o = w if origin is None else origin
        key = (o.untyped_storage().data_ptr(), o.storage_offset(), tuple(o.stride()), o._version, tuple(o.shape), pow2)
        if refresh or self.entries[g] is None or self.keys[g] != key:
            self.entries[g] = Q.block_quantize(w.detach(), with_transpose=True, pow2=pow2)
            self.keys[g] = key
            self.misses += 1
        else:
            self.hits += 1
        return self.entries[g]

    def clear(self) -> None:
        self.entries, self.keys = [], []


class _GroupedScaledFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sizes: Tuple[int, ...], pow2: bool, cache: WeightQuantCache, refresh: bool, fuse_wgrad: bool,
                origins, *weights):
        N = weights[0].shape[0]
        xq, xs = Q.tile_quantize(x, pow2)
        out = torch.empty(x.shape[0], N, dtype=x.dtype, device=x.device)
        wq = [cache.get(g, w, pow2, refresh, origins[g]) for g, w in enumerate(weights)]
        r = 0
        for g, n in enumerate(sizes):
            if n:
                Q.scaled_gemm(xq[r: r + n], xs[r: r + n], wq[g][0], wq[g][1], out=out[r: r + n])
            r += n
        ctx.save_for_backward(x, *weights)
        ctx.sizes, ctx.pow2, ctx.wq, ctx.fuse_wgrad = sizes, pow2, wq, fuse_wgrad
        ctx.w_refs = weights
        return out

    @staticmethod
    def backward(ctx, dy):
        x, *weights = ctx.saved_tensors
        dy = dy.contiguous()
        gq, gs = Q.tile_quantize(dy, ctx.pow2)
        dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
        dws: List[Optional[torch.Tensor]] = []
        r = 0
        for g, n in enumerate(ctx.sizes):
            w = weights[g]
            ref = ctx.w_refs[g]
            mg = getattr(ref, "main_grad", None) if ctx.fuse_wgrad else None
            if not ctx.needs_input_grad[7 + g]:
                dws.append(None)
            elif n == 0:
                dws.append(None if mg is not None else torch.zeros_like(w))
            else:
                q, s, qt = ctx.wq[g]
                if dx is not None:
                    Q.scaled_gemm(gq[r: r + n], gs[r: r + n], qt, s.t().contiguous(), out=dx[r: r + n])
                target = mg if mg is not None else torch.empty_like(w)
                if n % 128 == 0:
                    a, a_s = Q.tile_quantize_transposed(dy[r: r + n], ctx.pow2)
                    b, b_s = Q.tile_quantize_transposed(x[r: r + n], ctx.pow2)
                    Q.scaled_gemm(a, a_s, b, b_s, b_row_mode=True, out=target, accumulate=mg is not None)
                else:   # ragged group: the token dim cannot be cut into 128-strips
                    ops.gemm(dy[r: r + n], x[r: r + n], a_mn=True, b_mn=True, out=target, accumulate=mg is not None)
                if mg is not None:
                    ref.grad_added_to_main_grad = True
                    dws.append(None)
                else:
                    dws.append(target)
            if n and dx is not None and not ctx.needs_input_grad[7 + g]:
                q, s, qt = ctx.wq[g]
                Q.scaled_gemm(gq[r: r + n], gs[r: r + n], qt, s.t().contiguous(), out=dx[r: r + n])
            r += n
        return (dx, None, None, None, None, None, None, *dws)


_default_cache = {}


def grouped_scaled_linear(x: torch.Tensor, w: Union[torch.Tensor, Sequence[torch.Tensor]], sizes: Sequence[int],
                          pow2: bool = False, cache: Optional[WeightQuantCache] = None, refresh: bool = False,
                          fuse_wgrad_accumulation: bool = False) -> torch.Tensor:
    weights = list(w.unbind(0)) if isinstance(w, torch.Tensor) else list(w)
    N, K = weights[0].shape
    sizes = tuple(int(s) for s in sizes)
    if x.dtype != torch.bfloat16 or K % 128 or N % 128:
        r, outs = 0, []
        for g, n in enumerate(sizes):
            outs.append(ops.linear(x[r: r + n], weights[g].to(x.dtype)))
            r += n
        return torch.cat(outs)
    origins = weights
    # the kernels want contiguous bf16 operands; a transposed parameter view is copied (the copy is part of the
    # autograd graph), while the cache keeps recognising it by the parameter's own identity
    weights = [wg.to(torch.bfloat16) if wg.dtype != torch.bfloat16 else wg for wg in weights]
    weights = [wg if wg.is_contiguous() else wg.contiguous() for wg in weights]
    if cache is None:       # callers without a cache of their own: keyed by the first weight's storage and geometry
        w0 = origins[0]
        cache = _default_cache.setdefault((w0.untyped_storage().data_ptr(), w0.storage_offset(), tuple(w0.stride())),
                                          WeightQuantCache())
    return _GroupedScaledFn.apply(x, sizes, pow2, cache, refresh, fuse_wgrad_accumulation, origins, *weights)
