"""FP8 (e4m3) block-scaled quantisation: 1x128 tiles for activations / gradients, 128x128 blocks for
weights, each optionally emitting the transposed tensor quantised along its new reduction dim.
Scales are inverse scales (``x ~= q * s``, ``s = max(amax, eps) / 448``), optionally rounded up to a
power of two. CUDA kernels: csrc/fp8.cu; the ``*_reference`` functions are the PyTorch oracle/CPU path.
(Reference: atorch/modules/fp8/quantize.py:9-376, triton_kernel.py:21-141.)
"""
from __future__ import annotations

import ctypes
from enum import Enum
from typing import Optional, Tuple

import torch

from ... import _lib

FP8_MAX = 448.0
E4M3 = torch.float8_e4m3fn


class ScaleType(Enum):
    TENSORWISE = "tensorwise"
    AXISWISE = "axiswise"
    TILEWISE = "tilewise"
    BLOCKWISE = "blockwise"


def _scale(amax: torch.Tensor, pow2: bool) -> torch.Tensor:
    s = amax.float().clamp(min=1e-12) / FP8_MAX
    return torch.exp2(torch.ceil(torch.log2(s))) if pow2 else s


def tile_quantize_reference(x: torch.Tensor, pow2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    M, K = x.shape
    xt = x.float().view(M, K // 128, 128)
    s = _scale(xt.abs().amax(-1), pow2)
    q = (xt / s.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(E4M3).view(M, K)
    return q, s


def block_quantize_reference(w: torch.Tensor, pow2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    N, K = w.shape
    wb = w.float().view(N // 128, 128, K // 128, 128)
    s = _scale(wb.abs().amax((1, 3)), pow2)
    q = (wb / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(E4M3).view(N, K)
    return q, s


def dequantize_reference(q: torch.Tensor, s: torch.Tensor, block: bool) -> torch.Tensor:
    R, C = q.shape
    qf = q.float()
    if block:
        return (qf.view(R // 128, 128, C // 128, 128) * s[:, None, :, None]).view(R, C)
    return (qf.view(R, C // 128, 128) * s.unsqueeze(-1)).view(R, C)


def _use(x: torch.Tensor) -> bool:
    return _lib.use_kernels(x) and x.dtype == torch.bfloat16 and _lib.lib().has("atb_fp8_gemm")


def tile_quantize(x: torch.Tensor, pow2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [M, K] -> (q [M, K] e4m3, scales [M, K/128] fp32)."""
    M, K = x.shape
    if not _use(x) or K % 128:
        return tile_quantize_reference(x, pow2)
    x = x if x.stride(1) == 1 else x.contiguous()
    q = torch.empty(M, K, dtype=torch.uint8, device=x.device)
    s = torch.empty(M, K // 128, dtype=torch.float32, device=x.device)
    rc = _lib.lib().atb_fp8_tile_quant(_lib.ptr(x), _lib.ptr(q), _lib.ptr(s), ctypes.c_longlong(M), ctypes.c_int(K),
                                       ctypes.c_longlong(x.stride(0)), ctypes.c_int(int(pow2)), _lib.stream_ptr())
    _lib.check(rc, "atb_fp8_tile_quant")
    return q.view(E4M3), s


def tile_quantize_transposed(x: torch.Tensor, pow2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [M, K] -> (q_t [K, M] e4m3 quantised in strips of 128 along M, scales_t [K, M/128])."""
    M, K = x.shape
    if not _use(x) or M % 128 or K % 64:
        return tile_quantize_reference(x.t().contiguous(), pow2)
    x = x if x.stride(1) == 1 else x.contiguous()
    qt = torch.empty(K, M, dtype=torch.uint8, device=x.device)
    st = torch.empty(K, M // 128, dtype=torch.float32, device=x.device)
    rc = _lib.lib().atb_fp8_tile_quant_t(_lib.ptr(x), _lib.ptr(qt), _lib.ptr(st), ctypes.c_longlong(M),
                                         ctypes.c_int(K), ctypes.c_longlong(x.stride(0)), ctypes.c_int(int(pow2)),
                                         _lib.stream_ptr())
    _lib.check(rc, "atb_fp8_tile_quant_t")
    return qt.view(E4M3), st


def block_quantize(w: torch.Tensor, with_transpose: bool = False, pow2: bool = False):
    """w [N, K] -> (q [N, K], scales [N/128, K/128]) and, if asked, q_t [K, N] (scales_t = scales.t())."""
    N, K = w.shape
    if not _use(w) or N % 128 or K % 128:
        q, s = block_quantize_reference(w, pow2)
        return (q, s, q.t().contiguous()) if with_transpose else (q, s)
    w = w if w.stride(1) == 1 else w.contiguous()
    q = torch.empty(N, K, dtype=torch.uint8, device=w.device)
    qt = torch.empty(K, N, dtype=torch.uint8, device=w.device) if with_transpose else None
    s = torch.empty(N // 128, K // 128, dtype=torch.float32, device=w.device)
    rc = _lib.lib().atb_fp8_block_quant(_lib.ptr(w), _lib.ptr(q), _lib.ptr(qt), _lib.ptr(s), ctypes.c_int(N),
                                        ctypes.c_int(K), ctypes.c_longlong(w.stride(0)), ctypes.c_int(int(pow2)),
                                        _lib.stream_ptr())
    _lib.check(rc, "atb_fp8_block_quant")
    return (q.view(E4M3), s, qt.view(E4M3)) if with_transpose else (q.view(E4M3), s)


def dequantize(q: torch.Tensor, s: torch.Tensor, block: bool) -> torch.Tensor:
    R, C = q.shape
    if not (_lib.use_kernels(q) and _lib.lib().has("atb_fp8_dequant")) or C % 128:
        return dequantize_reference(q, s, block).to(torch.bfloat16)
    out = torch.empty(R, C, dtype=torch.bfloat16, device=q.device)
    rc = _lib.lib().atb_fp8_dequant(_lib.ptr(q), _lib.ptr(s.contiguous()), _lib.ptr(out), ctypes.c_longlong(R),
                                    ctypes.c_int(C), ctypes.c_int(int(block)), _lib.stream_ptr())
    _lib.check(rc, "atb_fp8_dequant")
    return out


def scaled_gemm_reference(aq, a_s, bq, b_s, b_row_mode: bool, out_dtype=torch.bfloat16):
    a = dequantize_reference(aq, a_s, False)
    b = dequantize_reference(bq, b_s, not b_row_mode)
    return (a @ b.t()).to(out_dtype)


def scaled_gemm(aq: torch.Tensor, a_s: torch.Tensor, bq: torch.Tensor, b_s: torch.Tensor, b_row_mode: bool = False,
                out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, accumulate: bool = False) -> torch.Tensor:
    """``C = sum_kb (A_q B_q^T)_kb * a_s[m, kb] * b_s[n/128 | n, kb]``; A_q [M, K], B_q [N, K] e4m3."""
    M, K = aq.shape
    N = bq.shape[0]
    if not (_lib.use_kernels(aq, bq) and _lib.lib().has("atb_fp8_gemm")) or K % 128 or N % 8 \
            or (not b_row_mode and N % 128):
        r = scaled_gemm_reference(aq, a_s, bq, b_s, b_row_mode, torch.float32)
        if out is not None:
            out.copy_((r + out.float()) if accumulate else r)
            return out
        return r.to(out_dtype)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=aq.device)
    rc = _lib.lib().atb_fp8_gemm(_lib.ptr(aq), _lib.ptr(bq), _lib.ptr(a_s.contiguous()), _lib.ptr(b_s.contiguous()),
                                 _lib.ptr(out), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                                 ctypes.c_longlong(out.stride(0)), ctypes.c_int(int(b_row_mode)),
                                 ctypes.c_int(int(out.dtype == torch.float32)), ctypes.c_int(int(accumulate)),
                                 _lib.stream_ptr(), _lib.ptr(_lib.status_word(aq.device)))
    _lib.check(rc, "atb_fp8_gemm")
    return out
