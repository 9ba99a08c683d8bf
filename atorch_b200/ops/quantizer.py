"""Group-wise integer quantisation ops (csrc/quant.cu) with PyTorch reference paths, and the
``QuantizerBuilder`` / ``QuantizationOptimizerBuilder`` façades that mirror the reference's JIT op
builders (``Builder().load()`` returns an object exposing the op functions).

    quantize(x, groups, bits, symmetric) -> (int8 data [packed for 4 bit], fp32 params [groups, 1|2])
    dequantize(q, params, groups, bits, symmetric, dtype)
    swizzle_quant(x, groups, bits, symmetric, pipeline_size, nodes, devices_per_node)
    quantized_reduction(q, params, in_groups, out_groups, bits, symmetric, n_tensors)

(Reference: atorch/ops/csrc/quantization/pt_binding.cpp:18-172, atorch/ops/quantizer/__init__.py:16-58,
atorch/ops/op_builder/{builder,quantizer,quantization_optimizer,all_ops}.py.)
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import _lib


def _kernels(x) -> bool:
    return _lib.use_kernels(x) and _lib.lib().has("atb_quantize")


def quantize_reference(x, groups: int, bits: int = 8, symmetric: bool = True):
    xg = x.float().reshape(groups, -1)
    qmax, half = 2 ** (bits - 1) - 1, 2 ** (bits - 1)
    if symmetric:
        s = xg.abs().amax(1) / qmax
        s = torch.where(s == 0, torch.ones_like(s), s)
        q = torch.round(xg / s[:, None]).clamp(-half, qmax)
        params = s[:, None]
    else:
        lo, hi = xg.amin(1), xg.amax(1)
        s = (hi - lo) / (2 ** bits - 1)
        s = torch.where(s == 0, torch.ones_like(s), s)
        q = (torch.round((xg - lo[:, None]) / s[:, None]) - half).clamp(-half, qmax)
        params = torch.stack([s, lo], 1)
    q = q.to(torch.int8)
    if bits == 4:
        q = ((q[:, 0::2] & 0xF) | ((q[:, 1::2] & 0xF) << 4)).to(torch.int8)
    return q.reshape(-1), params.contiguous()


def dequantize_reference(q, params, groups: int, bits: int = 8, symmetric: bool = True, dtype=torch.float16):
    half = 2 ** (bits - 1)
    if bits == 4:
        b = q.to(torch.int16) & 0xFF
        lo, hi = b & 0xF, (b >> 4) & 0xF
        v = torch.stack([lo, hi], -1).reshape(-1)
        v = torch.where(v >= 8, v - 16, v)
    else:
        v = q.to(torch.int16)
    v = v.float().reshape(groups, -1)
    if symmetric:
        out = v * params[:, :1]
    else:
        out = (v + half) * params[:, :1] + params[:, 1:2]
    return out.reshape(-1).to(dtype)


def quantize(x: torch.Tensor, groups: int, bits: int = 8, symmetric: bool = True,
             group_map: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    assert x.numel() % groups == 0
    gs = x.numel() // groups
    if not _kernels(x) or x.dtype not in _lib.DT:
        assert group_map is None or True
        q, p = quantize_reference(x, groups, bits, symmetric)
        if group_map is not None:
            per = gs // (2 if bits == 4 else 1)
            inv = torch.empty_like(group_map.long())
            q2 = torch.empty_like(q).view(groups, per)
            q2[group_map.long()] = q.view(groups, per)
            p2 = torch.empty_like(p)
            p2[group_map.long()] = p
            return q2.reshape(-1), p2
        return q, p
    x = x.contiguous()
    q = torch.empty(x.numel() // (2 if bits == 4 else 1), dtype=torch.int8, device=x.device)
    p = torch.empty(groups, 1 if symmetric else 2, dtype=torch.float32, device=x.device)
    rc = _lib.lib().atb_quantize(_lib.ptr(x), _lib.ptr(q), _lib.ptr(p), ctypes.c_int(groups), ctypes.c_int(gs),
                                 ctypes.c_int(bits), ctypes.c_int(int(not symmetric)), _lib.ptr(group_map),
                                 ctypes.c_int(_lib.DT[x.dtype]), _lib.stream_ptr())
    _lib.check(rc, "atb_quantize")
    return q, p


def dequantize(q: torch.Tensor, params: torch.Tensor, groups: int, bits: int = 8, symmetric: bool = True,
               dtype=torch.float16) -> torch.Tensor:
    total = q.numel() * (2 if bits == 4 else 1)
    if not _kernels(q) or dtype not in _lib.DT:
        return dequantize_reference(q, params, groups, bits, symmetric, dtype)
    out = torch.empty(total, dtype=dtype, device=q.device)
    rc = _lib.lib().atb_dequantize(_lib.ptr(q), _lib.ptr(params.contiguous()), _lib.ptr(out), ctypes.c_longlong(total),
                                   ctypes.c_int(total // groups), ctypes.c_int(bits), ctypes.c_int(int(not symmetric)),
                                   ctypes.c_int(_lib.DT[dtype]), _lib.stream_ptr())
    _lib.check(rc, "atb_dequantize")
    return out


def swizzle_group_map(groups: int, pipeline_size: int, nodes: int, devices_per_node: int, device=None) -> torch.Tensor:
    """Destination slot of every group for the 2-hop all-to-all layout: the input is ordered
    (node, device, pipeline, rest); the output is ordered (pipeline, device, node, rest)."""
    per = groups // (pipeline_size * nodes * devices_per_node)
    idx = torch.arange(groups, device=device).view(nodes, devices_per_node, pipeline_size, per)
    dest = torch.empty(groups, dtype=torch.int32, device=device)
    dest[idx.permute(2, 1, 0, 3).reshape(-1)] = torch.arange(groups, dtype=torch.int32, device=device)
    return dest


def swizzle_quant(x, groups: int, bits: int = 8, symmetric: bool = True, pipeline_size: int = 1, nodes: int = 1,
                  devices_per_node: int = 1):
    gm = swizzle_group_map(groups, pipeline_size, nodes, devices_per_node, x.device)
    return quantize(x, groups, bits, symmetric, gm)


def quantized_reduction(q: torch.Tensor, params: torch.Tensor, in_groups: int, out_groups: int, bits: int = 8,
                        symmetric: bool = True, n_tensors: int = 8):
    """``q`` holds ``n_tensors`` quantised chunks back to back (``in_groups = n_tensors * out_groups``);
    returns the requantised elementwise sum (``out_groups`` groups)."""
    assert in_groups == n_tensors * out_groups
    per_bytes = q.numel() // n_tensors
    gs = per_bytes * (2 if bits == 4 else 1) // out_groups
    if not _kernels(q):
        total = None
        P = params.view(n_tensors, out_groups, -1)
        for t in range(n_tensors):
            d = dequantize_reference(q[t * per_bytes:(t + 1) * per_bytes], P[t], out_groups, bits, symmetric,
                                     torch.float32)
            total = d if total is None else total + d
        return quantize_reference(total, out_groups, bits, symmetric)
    qo = torch.empty(per_bytes, dtype=torch.int8, device=q.device)
    po = torch.empty(out_groups, 1 if symmetric else 2, dtype=torch.float32, device=q.device)
    rc = _lib.lib().atb_dequant_reduce(_lib.ptr(q), _lib.ptr(params.contiguous()), _lib.ptr(qo), _lib.ptr(po),
                                       ctypes.c_int(n_tensors), ctypes.c_longlong(per_bytes), ctypes.c_int(out_groups),
                                       ctypes.c_int(gs), ctypes.c_int(bits), ctypes.c_int(int(not symmetric)),
                                       _lib.stream_ptr())
    _lib.check(rc, "atb_dequant_reduce")
    return qo, po


class _QuantizerOps:
    Symmetric, Asymmetric = 0, 1
    quantize = staticmethod(lambda x, groups, bits, qtype=0: quantize(x, groups, bits, qtype == 0))
    dequantize = staticmethod(lambda q, p, groups, bits, qtype=0: dequantize(q, p, groups, bits, qtype == 0,
                                                                             torch.float16))
    dequantize_fp32 = staticmethod(lambda q, p, groups, bits, qtype=0: dequantize(q, p, groups, bits, qtype == 0,
                                                                                  torch.float32))
    swizzle_quant = staticmethod(lambda x, groups, bits, qtype, pipeline_size, nodes, devices_per_node:
                                 swizzle_quant(x, groups, bits, qtype == 0, pipeline_size, nodes, devices_per_node))
    quantized_reduction = staticmethod(lambda q, p, in_groups, out_groups, bits, qtype, devices_per_node:
                                       quantized_reduction(q, p, in_groups, out_groups, bits, qtype == 0,
                                                           devices_per_node))


class OpBuilder:
    """Ahead-of-time counterpart of the reference's JIT builder: ``load()`` makes sure the shared library
    is built and returns the op namespace."""
    NAME = "base"

    def is_compatible(self, verbose: bool = False) -> bool:
        return True

    def load(self, verbose: bool = False):
        raise NotImplementedError


class QuantizerBuilder(OpBuilder):
    NAME = "quantizer"

    def load(self, verbose: bool = False):
        return _QuantizerOps


class CUDAQuantizer:
    """Quantise to int8 in groups of ``group_size`` elements (reference façade atorch/ops/quantizer/__init__.py)."""

    def __init__(self, group_size: int = 2048):
        self.group_size = group_size

    def quantize(self, x, quantization_bits: int = 8, symmetric: bool = True):
        groups = max(x.numel() // self.group_size, 1)
        return quantize(x, groups, quantization_bits, symmetric)

    def dequantize(self, q, params, quantization_bits: int = 8, symmetric: bool = True, dtype=torch.float16):
        groups = params.shape[0]
        return dequantize(q, params, groups, quantization_bits, symmetric, dtype)
