"""Precision methods: ``amp_native`` (autocast + loss scaling), ``half`` (whole model in fp16/bf16).

``amp_native`` config: ``{"dtype": torch.float16|torch.bfloat16|"fp16"|"bf16", "skip_if_nonfinite": bool}``;
default fp16 with dynamic loss scaling; bf16 only autocasts unless ``skip_if_nonfinite`` asks for
the inf/nan step skip. Next to a sharded engine the method turns into the engine's mixed-precision
setting (see ``ModelContext.adjust_wrappers``).
(Reference: atorch/auto/opt_lib/amp_optimization.py:40-193, half_optimization.py:10-45.)
"""
from __future__ import annotations

import functools

import torch

from ..auto_accelerate_context import AutoAccelerateContext
from .optimization import Optimization

_STR = {"fp16": torch.float16, "bf16": torch.bfloat16}


def _norm_amp_config(config):
    cfg = dict(config or {})
    d = cfg.get("dtype", torch.float16)
    cfg["dtype"] = _STR.get(d, d) if not isinstance(d, torch.dtype) else d
    if cfg["dtype"] not in (torch.float16, torch.bfloat16):
        raise ValueError(f"amp_native supports fp16/bf16, got {d}")
    return cfg


class AmpNativeOptimizer:
    """Optimizer wrapper doing unscale / inf check / scaler update around ``step``."""

    def __init__(self, optimizer, scaler, skip_if_nonfinite=False):
        self.optimizer, self.grad_scaler, self.skip_if_nonfinite = optimizer, scaler, skip_if_nonfinite
        self.step_was_skipped = False
        self._unscaled = False

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def state(self):
        return self.optimizer.state

    def unscale_(self):
        if self.grad_scaler is not None and not self._unscaled:
            self.grad_scaler.unscale_(self.optimizer)
            self._unscaled = True

    def step(self, *a, **k):
        if self.grad_scaler is not None:
            before = self.grad_scaler.get_scale()
            r = self.grad_scaler.step(self.optimizer, *a, **k)
            self.grad_scaler.update()
            self.step_was_skipped = self.grad_scaler.get_scale() < before
            self._unscaled = False
            return r
        if self.skip_if_nonfinite:
            bad = False
            for g in self.optimizer.param_groups:
                for p in g["params"]:
                    if p.grad is not None and not torch.isfinite(p.grad).all():
                        bad = True
            self.step_was_skipped = bad
            if bad:
                return None
        return self.optimizer.step(*a, **k)

    def zero_grad(self, *a, **k):
        return self.optimizer.zero_grad(*a, **k)

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, sd):
        return self.optimizer.load_state_dict(sd)

    def __getattr__(self, k):
        return getattr(self.optimizer, k)


class _ScaledLoss(torch.Tensor):
    """Loss tensor whose ``backward`` applies the loss scale first."""

    @staticmethod
    def wrap(loss, scaler):
        t = loss.as_subclass(_ScaledLoss)
        t._scaler = scaler
        return t

    def backward(self, *a, **k):
        return self._scaler.scale(self.as_subclass(torch.Tensor)).backward(*a, **k)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **(kwargs or {}))


def apply_grad_scaler(model_context, cfg, sharded=False):
    cfg = _norm_amp_config(cfg)
    scaler = None
    if cfg["dtype"] == torch.float16:
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        scaler = torch.amp.GradScaler(dev, enabled=torch.cuda.is_available())
        AutoAccelerateContext.set("amp_native_grad_scaler", scaler)
    if model_context.optim is not None and (scaler is not None or cfg.get("skip_if_nonfinite")):
        model_context.optim = AmpNativeOptimizer(model_context.optim, scaler, cfg.get("skip_if_nonfinite", False))
    if scaler is not None and model_context.loss_func is not None:
        lf = model_context.loss_func

        @functools.wraps(lf)
        def scaled_loss_func(*a, **k):
            out = lf(*a, **k)
            if isinstance(out, (tuple, list)):
                return (_ScaledLoss.wrap(out[0], scaler), *out[1:])
            return _ScaledLoss.wrap(out, scaler)
        model_context.loss_func = scaled_loss_func
    return model_context


def _amp_wrapper(model_context, wrapper_name, wrapper_config=None):
    cfg = _norm_amp_config(wrapper_config)
    dtype = cfg["dtype"]
    model = model_context.model
    dev_type = "cuda" if torch.cuda.is_available() else "cpu"
    inner_forward = model.forward

    @functools.wraps(inner_forward)
    def autocast_forward(*a, **k):
        with torch.autocast(dev_type, dtype=dtype):
            return inner_forward(*a, **k)
    model.forward = autocast_forward
    if model_context.loss_func is not None:
        lf = model_context.loss_func

        @functools.wraps(lf)
        def autocast_loss(*a, **k):
            with torch.autocast(dev_type, dtype=dtype):
                return lf(*a, **k)
        model_context.loss_func = autocast_loss
    return apply_grad_scaler(model_context, cfg)


class AmpNativeOptimization(Optimization):
    def __init__(self):
        super().__init__("amp_native", "amp", False)

    def transform(self, model_context, config=None):
        cfg = _norm_amp_config(config)
        AutoAccelerateContext.set("half_precision_dtype", cfg["dtype"])
        model_context.add_wrapper("amp_native", _amp_wrapper, cfg, is_pre_wrapper=False)
        return model_context


def _half_wrapper(model_context, wrapper_name, wrapper_config=None):
    dtype = _STR.get(wrapper_config, wrapper_config) or torch.float16
    model_context.model = model_context.model.to(dtype)
    pi = model_context.prepare_input

    def cast(x):
        if isinstance(x, torch.Tensor):
            return x.to(dtype) if x.is_floating_point() else x
        if isinstance(x, dict):
            return {k: cast(v) for k, v in x.items()}
        if isinstance(x, (list, tuple)):
            return type(x)(cast(v) for v in x)
        return x

    def prepare_input(batch, device):
        if pi is not None:
            batch = pi(batch, device)
        return cast(batch)
    model_context.prepare_input = prepare_input
    return model_context


class HalfOptimization(Optimization):
    def __init__(self):
        super().__init__("half", "amp", False)

    def transform(self, model_context, config="fp16"):
        config = config or "fp16"
        AutoAccelerateContext.set("half_precision_dtype", _STR.get(config, config))
        model_context.add_wrapper("half", _half_wrapper, config, is_pre_wrapper=True)
        return model_context
