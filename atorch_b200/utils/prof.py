"""``AProfiler``: per-module FLOPs / parameters / latency profile of one forward pass.

Forward pre/post hooks on every module record device time (CUDA events) and activation bytes;
FLOPs are counted analytically for the operator modules of this framework and torch (linear,
attention, embedding, norms, convolution) from input/output shapes. ``print_model_profile`` renders the
module tree down to ``module_depth`` with parameters, MACs, latency share; ``compute_gpu_utilization``
relates total FLOPs to the device peak (``GPUCapability``), i.e. hardware FLOPS utilisation.
(Reference: atorch/utils/prof.py:37-478,790-1206.)
"""
from __future__ import annotations

import time
from collections import OrderedDict
from typing import Dict, Optional

import torch
import torch.nn as nn

from ..common.constants import GPUCapability


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def module_flops(m: nn.Module, inputs, output) -> int:
    x = inputs[0] if inputs and isinstance(inputs[0], torch.Tensor) else None
    if isinstance(m, nn.Linear) and x is not None:
        return 2 * _numel(x.shape[:-1]) * m.in_features * m.out_features
    if isinstance(m, (nn.Conv1d, nn.Conv2d, nn.Conv3d)) and isinstance(output, torch.Tensor):
        k = _numel(m.kernel_size) * m.in_channels // m.groups
        return 2 * output.numel() * k
    if isinstance(m, (nn.LayerNorm, nn.GroupNorm)) and x is not None:
        return 5 * x.numel()
    if type(m).__name__ in ("RMSNorm", "AtorchRmsNorm") and x is not None:
        return 4 * x.numel()
    if type(m).__name__ == "FlashAttnModule" and len(inputs) >= 3:
        q, k = inputs[0], inputs[1]
        b, sq, h, d = q.shape
        f = 4 * b * h * sq * k.shape[1] * d
        return f // 2 if getattr(m, "causal", False) else f
    if isinstance(m, nn.MultiheadAttention) and x is not None:
        L = x.shape[0] if not m.batch_first else x.shape[1]
        B = x.numel() // (L * m.embed_dim)
        return 8 * B * L * m.embed_dim ** 2 + 4 * B * L * L * m.embed_dim
    return 0


class AProfiler:
    def __init__(self, model: nn.Module, profiling_depth: int = -1):
        self.model, self.depth = model, profiling_depth
        self.hooks, self.stats = [], OrderedDict()
        self.started = False
        self.total_duration = 0.0

    def start_profile(self, ignore_list=None) -> None:
        self.stats.clear()
        ignore = tuple(ignore_list or ())
        cuda = torch.cuda.is_available() and any(p.is_cuda for p in self.model.parameters())
        for name, m in self.model.named_modules():
            if isinstance(m, ignore):
                continue
            st = self.stats[name] = {"module": m, "flops": 0, "time": 0.0, "calls": 0, "act_bytes": 0,
                                     "params": sum(p.numel() for p in m.parameters(recurse=False)),
                                     "params_all": sum(p.numel() for p in m.parameters()), "depth": name.count(".") +
                                     (1 if name else 0)}

            def pre(mod, inp, _st=st):
                if cuda:
                    _st["_ev"] = torch.cuda.Event(enable_timing=True)
                    _st["_ev"].record()
                else:
                    _st["_t"] = time.time()

            def post(mod, inp, out, _st=st):
                if cuda:
                    e = torch.cuda.Event(enable_timing=True)
                    e.record()
                    _st.setdefault("_pairs", []).append((_st["_ev"], e))
                else:
                    _st["time"] += time.time() - _st["_t"]
                _st["flops"] += module_flops(mod, inp, out)
                _st["calls"] += 1
                if isinstance(out, torch.Tensor):
                    _st["act_bytes"] += out.numel() * out.element_size()
            self.hooks.append(m.register_forward_pre_hook(pre))
            self.hooks.append(m.register_forward_hook(post))
        self.started = True

    def stop_profile(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        for st in self.stats.values():
            for s, e in st.pop("_pairs", []):
                st["time"] += s.elapsed_time(e) / 1e3
        self.total_duration = self.stats.get("", {}).get("time", 0.0)

    def end_profile(self) -> None:
        for h in self.hooks:
            h.remove()
        self.hooks, self.started = [], False

    def get_total_flops(self) -> int:
        return sum(st["flops"] for st in self.stats.values())

    def get_total_params(self) -> int:
        return self.stats.get("", {}).get("params_all", sum(p.numel() for p in self.model.parameters()))

    def get_total_duration(self) -> float:
        return self.total_duration

    def _subtree_flops(self, name: str) -> int:
        pre = name + "." if name else ""
        return sum(st["flops"] for n, st in self.stats.items() if n == name or n.startswith(pre))

    def compute_gpu_utilization(self, batches_per_second: float, dtype: str = "bf16", backward: bool = True,
                                recompute: bool = False) -> float:
        """Hardware FLOPS utilisation for the profiled batch at the given rate."""
        if not torch.cuda.is_available():
            return 0.0
        peak = GPUCapability.peak(torch.cuda.get_device_name(), dtype) * 1e12
        mult = (4 if recompute else 3) if backward else 1
        return self.get_total_flops() * mult * batches_per_second / peak if peak else 0.0

    def print_model_profile(self, module_depth: int = -1, top_modules: int = 3, output_file: Optional[str] = None):
        lines = [f"params: {self.get_total_params():,}  fwd FLOPs: {self.get_total_flops():,}  "
                 f"fwd latency: {self.total_duration * 1e3:.3f} ms"]
        for name, st in self.stats.items():
            if module_depth >= 0 and st["depth"] > module_depth:
                continue
            share = st["time"] / self.total_duration * 100 if self.total_duration else 0.0
            lines.append(f"{'  ' * st['depth']}{name or type(self.model).__name__} ({type(st['module']).__name__}): "
                         f"params {st['params_all']:,}, FLOPs {self._subtree_flops(name):,}, "
                         f"latency {st['time'] * 1e3:.3f} ms ({share:.1f}%)")
        text = "\n".join(lines)
        if output_file:
            with open(output_file, "w") as f:
                f.write(text)
        else:
            print(text)
        return text


def report_device_memory(name: str = "") -> Dict[str, float]:
    if not torch.cuda.is_available():
        return {}
    free, total = torch.cuda.mem_get_info()
    return {"name": name, "allocated_mb": torch.cuda.memory_allocated() / 2 ** 20,
            "max_allocated_mb": torch.cuda.max_memory_allocated() / 2 ** 20,
            "reserved_mb": torch.cuda.memory_reserved() / 2 ** 20, "free_mb": free / 2 ** 20,
            "total_mb": total / 2 ** 20}
