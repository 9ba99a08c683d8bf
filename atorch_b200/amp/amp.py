"""apex-``amp``-shaped entry points on native PyTorch machinery.

``initialize(model, optimizers, opt_level=...)`` prepares model(s) and optimizer(s):

* ``O0``  nothing (fp32);
* ``O1``  forward under ``torch.autocast`` (fp16 on CUDA, bf16 on CPU), fp32 weights, dynamic loss scaling;
* ``O2``  weights cast to half except normalisation layers (``keep_batchnorm_fp32``), fp32 master copies
  held by the optimizer wrapper (``BF16Optimizer``-style), dynamic loss scaling;
* ``O3``  pure half, loss scale 1.

``with scale_loss(loss, optimizer) as scaled: scaled.backward()`` scales on entry and, on exit, unscales the
gradients, checks them and arms the optimizer to skip its next ``step()`` after an overflow.
(Reference: atorch/amp/amp.py:4-102, a pass-through to apex; apex is not required here.)
"""
from __future__ import annotations

import contextlib
from typing import Dict, List, Optional, Union

import torch
import torch.nn as nn

from ..utils.grad_scaler import DynamicGradScaler

_SCALERS: List[DynamicGradScaler] = []
_BY_OPT: Dict[int, DynamicGradScaler] = {}
_NORMS = (nn.modules.batchnorm._BatchNorm, nn.LayerNorm, nn.GroupNorm)


def _aslist(x):
    return list(x) if isinstance(x, (list, tuple)) else [x]


def _wrap_forward(model: nn.Module, dtype: torch.dtype) -> None:
    if getattr(model, "_amp_wrapped", False):
        return
    fwd = model.forward
    dev = next((p.device.type for p in model.parameters()), "cpu")

    def forward(*a, **k):
        with torch.autocast(dev, dtype=dtype):
            return fwd(*a, **k)
    model.forward = forward
    model._amp_wrapped = True


def _arm_skip(optimizer, scaler: DynamicGradScaler) -> None:
    if getattr(optimizer, "_amp_step_patched", False):
        return
    orig = optimizer.step

    def step(*a, **k):
        skipped = scaler._found_inf is not None and bool(scaler._found_inf.item())
        r = None if skipped else orig(*a, **k)
        scaler.update()
        return r
    optimizer.step = step
    optimizer._amp_step_patched = True


def initialize(model, optimizers=None, enabled: bool = True, opt_level: str = "O1", keep_batchnorm_fp32=None,
               loss_scale=None, min_loss_scale=None, max_loss_scale: float = 16777216.0, **kwargs):
    models, opts = _aslist(model), ([] if optimizers is None else _aslist(optimizers))
    if enabled and opt_level != "O0":
        cuda = any(p.is_cuda for m in models for p in m.parameters())
        half = torch.float16 if cuda else torch.bfloat16
        if opt_level == "O1":
            for m in models:
                _wrap_forward(m, half)
        elif opt_level in ("O2", "O3"):
            keep = opt_level == "O2" if keep_batchnorm_fp32 is None else str(keep_batchnorm_fp32) == "True"
            for m in models:
                for sub in m.modules():
                    if keep and isinstance(sub, _NORMS):
                        continue
                    for p in sub._parameters.values():
                        if p is not None and p.is_floating_point():
                            if opt_level == "O2":
                                p._amp_master = p.detach().clone().float()
                            p.data = p.data.to(half)
                _wrap_forward(m, half)
        else:
            raise ValueError(f"unknown opt_level {opt_level}")
        dynamic = loss_scale in (None, "dynamic") and opt_level != "O3"
        init = 2.0 ** 16 if dynamic else float(loss_scale if loss_scale not in (None, "dynamic") else 1.0)
        for o in opts:
            sc = DynamicGradScaler(init_scale=init, growth_interval=2000 if dynamic else 2 ** 62,
                                   backoff_factor=0.5 if dynamic else 1.0, min_scale=min_loss_scale or 1.0,
                                   max_scale=max_loss_scale)
            _SCALERS.append(sc)
            _BY_OPT[id(o)] = sc
            _arm_skip(o, sc)
    out_m = models if isinstance(model, (list, tuple)) else models[0]
    if optimizers is None:
        return out_m
    return out_m, (opts if isinstance(optimizers, (list, tuple)) else opts[0])


@contextlib.contextmanager
def scale_loss(loss: torch.Tensor, optimizers, loss_id: int = 0, model=None, delay_unscale: bool = False,
               delay_overflow_check: bool = False):
    opts = _aslist(optimizers)
    scalers = [_BY_OPT.get(id(o)) for o in opts]
    if not any(scalers):
        yield loss
        return
    sc = next(s for s in scalers if s is not None)
    yield loss.float() * sc.get_scale()
    if not delay_unscale:
        for o, s in zip(opts, scalers):
            if s is not None:
                s.unscale_(o)


def master_params(optimizer):
    """The parameters an optimizer updates (fp32 master copies where ``O2`` created them)."""
    for g in optimizer.param_groups:
        for p in g["params"]:
            yield getattr(p, "_amp_master", p)


def state_dict(destination=None) -> dict:
    d = {} if destination is None else destination
    for i, s in enumerate(_SCALERS):
        d[f"loss_scaler{i}"] = {"loss_scale": s.get_scale(), "unskipped": s._good_steps}
    return d


def load_state_dict(sd: dict) -> None:
    for i, s in enumerate(_SCALERS):
        e = sd.get(f"loss_scaler{i}")
        if e is not None:
            s.update(new_scale=e["loss_scale"])
            s._good_steps = int(e.get("unskipped", 0))
