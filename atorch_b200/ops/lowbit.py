"""Bit-packing of optimizer states (csrc/quant.cu): absmax-linear 8/16-bit codes and nonlinear
(table lookup) 4/8-bit codes with optional stochastic rounding, in groups of ``group_size`` elements.
(Reference: atorch/ops/csrc/quantization_optimizer/quantization_optimizer.cu:28-686 called from
atorch/optimizers/low_bit/functional.py:360-401.)
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from .. import _lib


def create_dynamic_map(signed: bool = True, bits: int = 8, power: float = 2.0) -> torch.Tensor:
    """Sorted code book in [-1, 1] (or [0, 1]) with ``2**bits`` entries, denser near zero."""
    n = 2 ** bits
    if signed:
        h = n // 2
        neg = -(torch.arange(h, 0, -1, dtype=torch.float32) / h) ** power          # -1 ... just below 0
        pos = (torch.arange(0, h, dtype=torch.float32) / (h - 1)) ** power         # 0 ... 1
        return torch.cat([neg, pos])
    return (torch.arange(0, n, dtype=torch.float32) / (n - 1)) ** power


def _k(x) -> bool:
    return _lib.use_kernels(x) and _lib.lib().has("atb_pack_linear")


def pack_absmax_linear(x: torch.Tensor, bits: int = 8, group_size: int = 2048) -> Tuple[torch.Tensor, torch.Tensor]:
    n = x.numel()
    groups = (n + group_size - 1) // group_size
    qmax = 127 if bits == 8 else 32767
    dt = torch.int8 if bits == 8 else torch.int16
    xf = x.reshape(-1).float().contiguous()
    if not _k(x):
        pad = groups * group_size - n
        xp = torch.nn.functional.pad(xf, (0, pad)).view(groups, group_size)
        am = xp.abs().amax(1)
        code = torch.round(xp * (qmax / am.clamp(min=1e-30))[:, None]).to(dt).reshape(-1)[:n]
        return code, am
    code = torch.empty(n, dtype=dt, device=x.device)
    am = torch.empty(groups, dtype=torch.float32, device=x.device)
    rc = _lib.lib().atb_pack_linear(_lib.ptr(xf), _lib.ptr(code), _lib.ptr(am), ctypes.c_longlong(n),
                                    ctypes.c_int(group_size), ctypes.c_int(bits), _lib.stream_ptr())
    _lib.check(rc, "atb_pack_linear")
    return code, am


def unpack_absmax_linear(code: torch.Tensor, absmax: torch.Tensor, bits: int = 8, group_size: int = 2048) -> torch.Tensor:
    n = code.numel()
    qmax = 127 if bits == 8 else 32767
    if not _k(code):
        g = torch.arange(n, device=code.device) // group_size
        return code.float() * absmax[g] / qmax
    out = torch.empty(n, dtype=torch.float32, device=code.device)
    rc = _lib.lib().atb_unpack_linear(_lib.ptr(code), _lib.ptr(absmax), _lib.ptr(out), ctypes.c_longlong(n),
                                      ctypes.c_int(group_size), ctypes.c_int(bits), _lib.stream_ptr())
    _lib.check(rc, "atb_unpack_linear")
    return out


def pack_nonlinear(x: torch.Tensor, qmap: torch.Tensor, bits: int = 4, group_size: int = 128,
                   stochastic: bool = False, seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    n = x.numel()
    groups = (n + group_size - 1) // group_size
    xf = x.reshape(-1).float().contiguous()
    if not _k(x):
        pad = groups * group_size - n
        xp = torch.nn.functional.pad(xf, (0, pad)).view(groups, group_size)
        am = xp.abs().amax(1)
        v = (xp / am.clamp(min=1e-30)[:, None]).reshape(-1)
        qm = qmap.to(v.device)
        lo = (torch.bucketize(v, qm, right=True) - 1).clamp(0, qm.numel() - 1)
        hi = (lo + 1).clamp(max=qm.numel() - 1)
        a, b = qm[lo], qm[hi]
        if stochastic:
            g = torch.Generator(device="cpu").manual_seed(seed)
            u = torch.rand(v.shape, generator=g).to(v.device)
            up = (v - a) > u * (b - a)
        else:
            up = (v - a) > (b - v)
        c = torch.where(up & (hi > lo), hi, lo).to(torch.uint8)
        if bits == 4:
            c = (c[0::2] | (c[1::2] << 4))
            return c[: (n + 1) // 2], am
        return c[:n], am
    code = torch.zeros(n if bits == 8 else (groups * group_size) // 2, dtype=torch.uint8, device=x.device)
    am = torch.empty(groups, dtype=torch.float32, device=x.device)
    rc = _lib.lib().atb_pack_nonlinear(_lib.ptr(xf), _lib.ptr(code), _lib.ptr(am),
                                       _lib.ptr(qmap.to(x.device).float().contiguous()), ctypes.c_longlong(n),
                                       ctypes.c_int(group_size), ctypes.c_int(bits), ctypes.c_int(int(stochastic)),
                                       ctypes.c_ulonglong(seed), _lib.stream_ptr())
    _lib.check(rc, "atb_pack_nonlinear")
    return code, am


def unpack_nonlinear(code: torch.Tensor, absmax: torch.Tensor, qmap: torch.Tensor, n: int, bits: int = 4,
                     group_size: int = 128) -> torch.Tensor:
    if not _k(code):
        if bits == 4:
            c = torch.stack([code & 0xF, code >> 4], -1).reshape(-1)[:n].long()
        else:
            c = code[:n].long()
        g = torch.arange(n, device=code.device) // group_size
        return qmap.to(code.device)[c] * absmax[g]
    out = torch.empty(n, dtype=torch.float32, device=code.device)
    rc = _lib.lib().atb_unpack_nonlinear(_lib.ptr(code), _lib.ptr(absmax), _lib.ptr(qmap.to(code.device).float().contiguous()),
                                         _lib.ptr(out), ctypes.c_longlong(n), ctypes.c_int(group_size),
                                         ctypes.c_int(bits), _lib.stream_ptr())
    _lib.check(rc, "atb_unpack_nonlinear")
    return out


class QuantizationOptimizerBuilder:
    NAME = "quantization_optimizer"

    def is_compatible(self, verbose: bool = False) -> bool:
        return True

    def load(self, verbose: bool = False):
        import types

        return types.SimpleNamespace(pack_absmax_linear=pack_absmax_linear, unpack_absmax_linear=unpack_absmax_linear,
                                     pack_nonlinear=pack_nonlinear, unpack_nonlinear=unpack_nonlinear)
