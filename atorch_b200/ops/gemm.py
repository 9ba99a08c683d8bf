"""bf16 GEMM on the tcgen05 tensor cores and the autograd ``linear`` built on it.

``gemm`` computes ``C (+)= alpha * op(A) @ op(B)^T (+ bias)`` with either operand stored K-major or
MN-major, so that the forward, dgrad and wgrad products of a linear layer all read their operands
as they lie in memory. On a CPU-only machine the same function evaluates the product with PyTorch
(the reference implementation that the GPU tests compare against).

``linear`` is the drop-in for ``torch.nn.functional.linear`` used by every projection of the models
in this package. Its backward accumulates the weight gradient straight into ``weight.main_grad``
when the parameter carries such a buffer (the flat gradient buffers of the sharded data-parallel
engines), which removes the separate gradient tensor and the accumulate pass.

Reference counterpart: cuBLAS behind ``nn.Linear`` (atorch/modules/distributed_modules/layers.py:117-151).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import _lib


# CTA-pair kernel (tcgen05 cta_group::2, 256x256 tiles) for problems with M, N >= 256
PAIR_KERNEL_DEFAULT = os.environ.get("ATB_GEMM_PAIR", "1") == "1"


def _pitch(t: torch.Tensor) -> int:
    return t.stride(0) if t.dim() == 2 else t.shape[-1]


def gemm_reference(a, b, a_mn=False, b_mn=False, out=None, out_dtype=None, accumulate=False, alpha=1.0, bias=None):
    """fp32-accumulated PyTorch evaluation of the same contract (the oracle for the kernel)."""
    A = a.t() if a_mn else a
    B = b.t() if b_mn else b
    r = (A.float() @ B.float().t()) * alpha
    if bias is not None:
        r = r + bias.float()
    if out is not None:
        if accumulate:
            r = r + out.float()
        out.copy_(r.to(out.dtype))
        return out
    return r.to(out_dtype or a.dtype)


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_mn: bool = False,
    b_mn: bool = False,
    out: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
    accumulate: bool = False,
    alpha: float = 1.0,
    bias: Optional[torch.Tensor] = None,
    tile_n: int = 0,
    max_ctas: int = 0,
    kernel: str = "auto",
    residual: Optional[torch.Tensor] = None,
    groups: Optional[dict] = None,
) -> torch.Tensor:
    """``out[M,N] (+)= alpha * A[M,K] @ B[N,K]^T (+ bias[N])``.

    ``a`` is stored ``[M,K]`` (or ``[K,M]`` when ``a_mn``), ``b`` is stored ``[N,K]`` (or ``[K,N]``
    when ``b_mn``). Inputs are bf16, accumulation is fp32, the output is bf16 or fp32.

    ``groups`` (mixture-of-experts buffers, CTA-pair kernel only): ``{"counts": int32 device tensor,
    "m_rows": r}`` - rows of A come in groups of ``r`` slots (a multiple of 256) of which only the first
    ``counts[g]`` hold data and the rest is zero: tiles beyond the count are not computed, their output is
    zero. ``"k_rows": r`` - the same along the reduction dim (multiple of 64): empty k-blocks are skipped.
    ``"n_b": E, "bm_rows": R`` - ``b`` holds E stacked operands and rows ``[e*R, (e+1)*R)`` of A use the
    e-th (one launch for all local experts).
    """
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    n_b = int(groups.get("n_b", 1)) if groups else 1
    if n_b > 1:                      # stacked B operands: [E*N, K] (or [E*K, N] when b_mn)
        if b_mn:
            Kb //= n_b
        else:
            N //= n_b
    assert K == Kb, f"reduction dims differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
        assert not accumulate
    if not _lib.use_kernels(a, b, out) or a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or (N % 8) or (K % 8) or (M % 8):
        if n_b > 1:                  # reference: one product per stacked operand (inputs are zero beyond the counts)
            R = groups["bm_rows"]
            for e in range(n_b):
                be = b[e * K: (e + 1) * K] if b_mn else b[e * N: (e + 1) * N]
                gemm_reference(a[e * R: (e + 1) * R], be, a_mn, b_mn, out[e * R: (e + 1) * R], None, accumulate,
                               alpha, bias)
            return out
        r = gemm_reference(a, b, a_mn, b_mn, out, None, accumulate, alpha, bias)
        if residual is not None:
            r.add_(residual.to(r.dtype))
        return r
    if a.stride(-1) != 1:
        a = a.contiguous()
    if b.stride(-1) != 1:
        b = b.contiguous()
    assert out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    L = _lib.lib()
    use_pair = kernel == "2cta" or (kernel == "auto" and PAIR_KERNEL_DEFAULT and M >= 256 and N >= 256)
    if groups is not None:
        counts = groups.get("counts")
        assert counts is None or (counts.dtype == torch.int32 and counts.is_cuda)
        rc = L.atb_gemm_bf16_2cta_grouped(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias),
            ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
            ctypes.c_longlong(_pitch(a)), ctypes.c_longlong(_pitch(b)), ctypes.c_longlong(_pitch(out)),
            ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)),
            ctypes.c_int(int(out.dtype == torch.float32)), ctypes.c_int(int(accumulate)),
            ctypes.c_float(alpha), ctypes.c_int(tile_n), ctypes.c_int(max_ctas), _lib.ptr(residual),
            ctypes.c_longlong(_pitch(residual) if residual is not None else 0), _lib.ptr(counts),
            ctypes.c_int(int(groups.get("m_rows", 0))), ctypes.c_int(int(groups.get("k_rows", 0))),
            ctypes.c_int((K if b_mn else N) if n_b > 1 else 0), ctypes.c_int(int(groups.get("bm_rows", 0))),
            ctypes.c_int(n_b), _lib.stream_ptr(), _lib.ptr(_lib.status_word(a.device)))
        _lib.check(rc, f"atb_gemm_bf16_2cta_grouped M={M} N={N} K={K}")
        return out
    if use_pair:
        rc = L.atb_gemm_bf16_2cta(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias),
            ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
            ctypes.c_longlong(_pitch(a)), ctypes.c_longlong(_pitch(b)), ctypes.c_longlong(_pitch(out)),
            ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)),
            ctypes.c_int(int(out.dtype == torch.float32)), ctypes.c_int(int(accumulate)),
            ctypes.c_float(alpha), ctypes.c_int(tile_n), ctypes.c_int(max_ctas), _lib.ptr(residual),
            ctypes.c_longlong(_pitch(residual) if residual is not None else 0), _lib.stream_ptr(),
            _lib.ptr(_lib.status_word(a.device)))
        _lib.check(rc, f"atb_gemm_bf16_2cta M={M} N={N} K={K}")
        return out
    rc = L.atb_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_longlong(_pitch(a)), ctypes.c_longlong(_pitch(b)), ctypes.c_longlong(_pitch(out)),
        ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)),
        ctypes.c_int(int(out.dtype == torch.float32)), ctypes.c_int(int(accumulate)),
        ctypes.c_float(alpha), ctypes.c_int(tile_n), ctypes.c_int(max_ctas), _lib.ptr(residual),
        ctypes.c_longlong(_pitch(residual) if residual is not None else 0),
        _lib.stream_ptr(), _lib.ptr(_lib.status_word(a.device)),
    )
    _lib.check(rc, f"atb_gemm_bf16 M={M} N={N} K={K}")
    return out


def _linear_grads(ctx, dy2, x2, weight, need_dx, need_dw):
    """dx and dW of ``y = x W^T`` from ``dy``; dW goes straight into ``weight.main_grad`` when there is one."""
    dx = dw = None
    if need_dx:
        dx = gemm(dy2, weight, b_mn=True, out_dtype=x2.dtype).view(ctx.x_shape)
    if need_dw:
        mg = getattr(ctx.weight_ref, "main_grad", None)
        if mg is not None:
            first = getattr(ctx.weight_ref, "_atb_first", False)     # untouched buffer: overwrite, no zero fill
            gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=not first)
            ctx.weight_ref._atb_first = False
            ctx.weight_ref.grad_added_to_main_grad = True
        else:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
    return dx, dw


def gemm_swiglu(x2: torch.Tensor, weight: torch.Tensor, keep_gate_up: bool):
    """``act = silu(x Wg^T) * (x Wu^T)`` for the fused weight ``[Wg; Wu]`` in one kernel (gated epilogue of the
    CTA-pair GEMM); with ``keep_gate_up`` also the bf16 gate|up tensor ``[T, 2F]`` that the backward needs."""
    T, K = x2.shape
    F = weight.shape[0] // 2
    act = torch.empty(T, F, dtype=x2.dtype, device=x2.device)
    gu = torch.empty(T, 2 * F, dtype=x2.dtype, device=x2.device) if keep_gate_up else None
    rc = _lib.lib().atb_gemm_bf16_2cta_swiglu(
        _lib.ptr(x2), _lib.ptr(weight), _lib.ptr(act), _lib.ptr(gu), ctypes.c_int(T), ctypes.c_int(F), ctypes.c_int(K),
        ctypes.c_longlong(_pitch(x2)), ctypes.c_longlong(_pitch(weight)), ctypes.c_longlong(F),
        ctypes.c_longlong(2 * F), _lib.stream_ptr(), _lib.ptr(_lib.status_word(x2.device)))
    _lib.check(rc, f"atb_gemm_bf16_2cta_swiglu T={T} F={F} K={K}")
    return act, gu


class _LinearSwiGLU(torch.autograd.Function):
    """``swiglu(x @ W^T)`` with the activation computed in the GEMM epilogue. A pass that needs no gradient (the
    first pass of an activation-checkpointed block) never writes the ``[T, 2F]`` pre-activation; a pass that does
    writes it from the same epilogue, so the separate SwiGLU kernel and its read of that tensor disappear."""

    @staticmethod
    def forward(ctx, x, weight):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
        need = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        act, gu = gemm_swiglu(x2, weight, need)
        if need:
            ctx.save_for_backward(x2, weight, gu)
        ctx.x_shape, ctx.weight_ref = shp, weight
        return act.view(*shp[:-1], act.shape[-1])

    @staticmethod
    def backward(ctx, dact):
        from .elementwise import swiglu_backward

        x2, weight, gu = ctx.saved_tensors
        dgu = swiglu_backward(gu, dact.reshape(-1, dact.shape[-1]))
        dx, dw = _linear_grads(ctx, dgu, x2, weight, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return dx, dw


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` for ``weight = [Wg; Wu]`` (``[2F, K]``), the gated MLP's first half."""
    from .elementwise import swiglu

    F = weight.shape[0] // 2
    if not (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and _lib.use_kernels(x, weight)
            and _lib.lib().has("atb_gemm_bf16_2cta_swiglu") and F % 8 == 0 and x.shape[-1] % 8 == 0
            and weight.stride(-1) == 1 and PAIR_KERNEL_DEFAULT):
        return swiglu(linear(x, weight))
    return _LinearSwiGLU.apply(x, weight)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.x_shape = shp
        ctx.weight_ref = weight
        if residual is not None:
            # out = residual + x W^T : the epilogue reads the residual stream and adds it before the store
            r2 = residual.reshape(-1, weight.shape[0])
            r2 = r2 if r2.stride(-1) == 1 else r2.contiguous()
            out = gemm(x2, weight, bias=bias, out_dtype=x.dtype, residual=r2)
        else:
            out = gemm(x2, weight, bias=bias, out_dtype=x.dtype)
        return out.view(*shp[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        db = dres = None
        dx, dw = _linear_grads(ctx, dy2, x2, weight, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy
        return dx, dw, db, dres


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``residual + x @ weight.T + bias`` with the tcgen05 GEMM in forward, dgrad and wgrad."""
    if x.dtype != torch.bfloat16 or not _lib.use_kernels(x, weight):
        y = torch.nn.functional.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
        return y if residual is None else residual + y
    return _Linear.apply(x, weight, bias, residual)
