"""``ATorchGroupedLinear``: ``num_gemms`` linears (``weight{i}`` of shape ``[out, in]``) applied to the
row groups of one input, ``forward(inp, m_splits, is_first_microbatch=None)``.

With ``fp8`` on, all three GEMM families run block-scaled e4m3. The quantised weights live in a
``WeightQuantCache``: ``is_first_microbatch=True`` (or ``None``) quantises them, ``is_first_microbatch=False``
reuses what the first micro-batch of the step produced (unless ``FORCE_QUANTIZE_PER_MICROBATCH`` is set or a
weight changed in between). ``fuse_wgrad_accumulation`` adds weight gradients into ``weight{i}.main_grad``
and returns no ``.grad``.
(Reference: atorch/modules/fp8/quantized_grouped_linear.py:36-584.)
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.nn as nn

from ... import ops
from ...ops import moe as moe_ops
from .grouped import WeightQuantCache, grouped_scaled_linear


class ATorchGroupedLinear(nn.Module):
    def __init__(self, num_gemms: int, in_features: int, out_features: int, bias: bool = False,
                 params_dtype=torch.bfloat16, device=None, fp8: bool = True, fuse_wgrad_accumulation: bool = False,
                 sequence_parallel: bool = False, init_method=None, **kwargs):
        super().__init__()
        self.num_gemms, self.in_features, self.out_features = num_gemms, in_features, out_features
        self.fp8, self.fuse_wgrad_accumulation, self.sequence_parallel = fp8, fuse_wgrad_accumulation, sequence_parallel
        self.use_bias = bias
        for i in range(num_gemms):
            w = nn.Parameter(torch.empty(out_features, in_features, dtype=params_dtype, device=device))
            (init_method or (lambda t: nn.init.normal_(t, std=0.02)))(w)
            self.register_parameter(f"weight{i}", w)
            if bias:
                self.register_parameter(f"bias{i}", nn.Parameter(torch.zeros(out_features, dtype=params_dtype,
                                                                           device=device)))
        self.force_requantize = os.environ.get("FORCE_QUANTIZE_PER_MICROBATCH", "0") in ("1", "true", "True")
        self.quant_cache = WeightQuantCache()

    def weights(self) -> List[torch.Tensor]:
        return [getattr(self, f"weight{i}") for i in range(self.num_gemms)]

    def forward(self, inp: torch.Tensor, m_splits: List[int], is_first_microbatch: Optional[bool] = None):
        assert len(m_splits) == self.num_gemms and sum(m_splits) == inp.shape[0]
        if self.fp8 and inp.dtype == torch.bfloat16:
            refresh = self.force_requantize or is_first_microbatch is None or bool(is_first_microbatch)
            out = grouped_scaled_linear(inp, self.weights(), m_splits, cache=self.quant_cache, refresh=refresh,
                                        fuse_wgrad_accumulation=self.fuse_wgrad_accumulation)
        else:
            out = moe_ops.grouped_gemm(inp, torch.stack(self.weights()).to(inp.dtype), m_splits, trans_b=True)
        if self.use_bias:
            idx = torch.repeat_interleave(torch.arange(self.num_gemms, device=inp.device),
                                          torch.tensor(m_splits, device=inp.device))
            b = torch.stack([getattr(self, f"bias{i}") for i in range(self.num_gemms)])
            out = ops.bias_gather_add(out, b.to(out.dtype), idx)
        return out
