"""Helpers around fp8 modules (reference: atorch/modules/fp8/utils.py:17-118)."""
from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.nn as nn

from .precision_switchable_linear import PrecisionSwitchableLinear
from .scaled_linear import ScaledLinear, fp8_shapes_ok


def _match(name: str, include: Optional[Iterable[str]], exclude: Optional[Iterable[str]]) -> bool:
    if include and not any(s in name for s in include):
        return False
    if exclude and any(s in name for s in exclude):
        return False
    return True


def convert_linears_to_fp8(model: nn.Module, config: dict) -> int:
    """Replace eligible ``nn.Linear`` modules (name include/exclude filters, dims divisible by the
    scale block) by ``ScaledLinear`` or ``PrecisionSwitchableLinear``; returns the count."""
    include, exclude = config.get("include"), config.get("exclude")
    switchable = bool(config.get("precision_switchable", False))
    kw = {}
    if config.get("scale_method"):
        kw["scale_method"] = config["scale_method"]
    n = 0
    for pname, parent in list(model.named_modules()):
        for cname, child in list(parent._modules.items()):
            full = f"{pname}.{cname}" if pname else cname
            if type(child) is nn.Linear and _match(full, include, exclude) and \
                    fp8_shapes_ok(child.in_features, child.out_features):
                cls = PrecisionSwitchableLinear if switchable else ScaledLinear
                parent._modules[cname] = cls.from_linear(child, **kw)
                n += 1
    if config.get("verbose"):
        print(f"fp8: converted {n} linear modules")
    return n


def set_linear_modules_precision(model: nn.Module, fp8_include_name_pattern=None, fp8_exclude_name_pattern=None,
                                 precision: str = "fp8", verbose: bool = False) -> int:
    import re

    n = 0
    for name, m in model.named_modules():
        if isinstance(m, PrecisionSwitchableLinear):
            if fp8_include_name_pattern and not re.search(fp8_include_name_pattern, name):
                continue
            if fp8_exclude_name_pattern and re.search(fp8_exclude_name_pattern, name):
                continue
            m.switch_precision(precision)
            n += 1
    return n


def get_fp8_module_count(model: nn.Module):
    """(fp8 modules, fp8-capable modules currently in original precision, plain linears)."""
    fp8 = orig = plain = 0
    for m in model.modules():
        if isinstance(m, ScaledLinear):
            if m.use_fp8:
                fp8 += 1
            else:
                orig += 1
        elif isinstance(m, nn.Linear):
            plain += 1
    return fp8, orig, plain


def get_fp8_quantize_underflows(x: torch.Tensor) -> float:
    """Fraction of non-zero entries that become zero under 1x128 e4m3 quantisation."""
    from .quantize import dequantize_reference, tile_quantize_reference

    K = x.shape[-1] // 128 * 128
    x2 = x.reshape(-1, x.shape[-1])[:, :K]
    q, s = tile_quantize_reference(x2)
    back = dequantize_reference(q, s, False)
    nz = x2 != 0
    return float(((back == 0) & nz).sum()) / max(int(nz.sum()), 1)
