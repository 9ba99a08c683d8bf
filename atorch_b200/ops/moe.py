"""Token permutation for mixture-of-experts and the grouped GEMM that consumes it.

``permute(tokens, expert_idx)``: stable sort of the flattened ``[T, k]`` expert ids; row j of the result
is token ``sorted[j] // k``. ``unpermute`` scatters expert outputs back, weights them with the routing
probabilities and sums over the k choices. Counts per expert stay on the device
(``tokens_per_expert``), the host only learns them when a variable-size exchange needs split lists.

``grouped_gemm(x, w, batch_sizes, trans_b)``: consecutive row groups of ``x`` times one weight per
group, each product on the tcgen05 GEMM (``ops.gemm``) with its forward / dgrad / wgrad layouts.
(Reference semantics: atorch/modules/moe/token_dispatcher.py:89-161; grouped_gemm.ops.gmm used at
atorch/modules/moe/grouped_gemm_moe.py:841-850; megablocks sort/histogram ops at :566-596.)
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .gemm import gemm, linear


def tokens_per_expert(expert_idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """int64 histogram ``[num_experts]`` of the routed expert ids (device resident, deterministic)."""
    return torch.bincount(expert_idx.reshape(-1), minlength=num_experts)


def permute(tokens: torch.Tensor, expert_idx: torch.Tensor, num_out_tokens: Optional[int] = None
            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """tokens ``[T, H]``, expert_idx ``[T, k]`` (or ``[T]``) -> (permuted ``[T*k, H]``, sorted_indices)."""
    k = expert_idx.shape[1] if expert_idx.dim() > 1 else 1
    flat = expert_idx.reshape(-1)
    sorted_idx = torch.argsort(flat, stable=True)
    if num_out_tokens is not None:
        sorted_idx = sorted_idx[:num_out_tokens]
    return tokens.index_select(0, sorted_idx // k), sorted_idx


def unpermute(permuted: torch.Tensor, sorted_idx: torch.Tensor, probs: Optional[torch.Tensor] = None,
              topk: int = 1, num_tokens: Optional[int] = None) -> torch.Tensor:
    """Inverse of :func:`permute`: ``[T*k, H] -> [T, H]`` with optional prob-weighted sum over k."""
    n_slots = (num_tokens * topk) if num_tokens is not None else (probs.numel() if probs is not None
                                                                   else sorted_idx.numel())
    out = torch.zeros(n_slots, permuted.shape[-1], dtype=permuted.dtype, device=permuted.device)
    out = out.index_copy(0, sorted_idx, permuted)
    out = out.view(-1, topk, permuted.shape[-1])
    if probs is not None:
        out = out * probs.view(-1, topk, 1).to(out.dtype)
    return out.sum(dim=1)


class _GroupedLinear(torch.autograd.Function):
    """y[g] = x[g] @ W[g]^T for consecutive row groups (W stored [G, N, K])."""

    @staticmethod
    def forward(ctx, x, w, sizes: Tuple[int, ...]):
        ctx.sizes = sizes
        ctx.save_for_backward(x, w)
        out = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
        r = 0
        for g, n in enumerate(sizes):
            if n:
                gemm(x[r: r + n], w[g], out=out[r: r + n])
            r += n
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        mg = getattr(w, "main_grad", None)
        dw = mg if mg is not None else torch.zeros_like(w)
        r = 0
        for g, n in enumerate(ctx.sizes):
            if n:
                gemm(dy[r: r + n], w[g], b_mn=True, out=dx[r: r + n])
                gemm(dy[r: r + n], x[r: r + n], a_mn=True, b_mn=True, out=dw[g], accumulate=mg is not None)
            r += n
        if mg is not None:
            w.grad_added_to_main_grad = True
            return dx, None, None
        return dx, dw, None


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, batch_sizes, trans_b: bool = False) -> torch.Tensor:
    """``gmm``: rows of ``a`` are split by ``batch_sizes`` (CPU ints / tensor); group g is multiplied by
    ``b[g]`` (``[K, N]``) or ``b[g]^T`` when ``trans_b`` (``[N, K]``)."""
    sizes = tuple(int(s) for s in (batch_sizes.tolist() if isinstance(batch_sizes, torch.Tensor) else batch_sizes))
    assert sum(sizes) == a.shape[0], "batch_sizes must cover all rows"
    if trans_b:
        return _GroupedLinear.apply(a, b, sizes)
    return _GroupedLinear.apply(a, b.transpose(1, 2).contiguous(), sizes)
