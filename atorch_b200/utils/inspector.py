"""``TensorInspector``: hooks that log statistics of activations and gradients of chosen modules (mean, std,
abs-max, fraction of zeros / non-finite values) and, for fp8 studies, the cosine similarity between a tensor
and its fp8 quantise-dequantise image. (Reference: atorch/utils/inspector/hooks.py:44-588.)"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn


def tensor_stats(t: torch.Tensor) -> Dict[str, float]:
    f = t.detach().float()
    finite = torch.isfinite(f)
    g = f[finite] if finite.any() else f.new_zeros(1)
    return {"mean": g.mean().item(), "std": g.std().item() if g.numel() > 1 else 0.0, "absmax": g.abs().max().item(),
            "zero_frac": (f == 0).float().mean().item(), "nonfinite_frac": 1.0 - finite.float().mean().item()}


def fp8_cosine_similarity(t: torch.Tensor) -> float:
    from ..modules.fp8.quantize import dequantize_reference, tile_quantize_reference

    K = t.shape[-1] // 128 * 128
    if K == 0:
        return 1.0
    x = t.detach().float().reshape(-1, t.shape[-1])[:, :K]
    q, s = tile_quantize_reference(x)
    y = dequantize_reference(q, s, False)
    return torch.nn.functional.cosine_similarity(x.reshape(1, -1), y.reshape(1, -1)).item()


class TensorInspector:
    def __init__(self, model: nn.Module, module_filter: Optional[Callable[[str, nn.Module], bool]] = None,
                 log_fn: Optional[Callable[[dict], None]] = None, with_fp8: bool = False, interval: int = 1):
        self.model, self.filter, self.with_fp8, self.interval = model, module_filter, with_fp8, interval
        self.records: List[dict] = []
        self.log_fn = log_fn or self.records.append
        self.hooks, self.step = [], 0

    def register(self) -> "TensorInspector":
        for name, m in self.model.named_modules():
            if self.filter is not None and not self.filter(name, m):
                continue
            self.hooks.append(m.register_forward_hook(self._fwd(name)))
            self.hooks.append(m.register_full_backward_hook(self._bwd(name)))
        return self

    def remove(self) -> None:
        for h in self.hooks:
            h.remove()
        self.hooks = []

    def _emit(self, name, kind, t):
        if self.step % self.interval:
            return
        rec = dict(tensor_stats(t), module=name, kind=kind, step=self.step)
        if self.with_fp8 and t.dim() >= 2:
            rec["fp8_cos"] = fp8_cosine_similarity(t)
        self.log_fn(rec)

    def _fwd(self, name):
        def fn(mod, inp, out):
            if isinstance(out, torch.Tensor):
                self._emit(name, "activation", out)
        return fn

    def _bwd(self, name):
        def fn(mod, gin, gout):
            if gout and isinstance(gout[0], torch.Tensor):
                self._emit(name, "grad_output", gout[0])
        return fn

    def next_step(self) -> None:
        self.step += 1
