"""``checkpoint``: activation recomputation for chosen module classes.

Config: a class / tuple of classes or class names, or a dict ``{"wrap_class": ..., "no_reentrant":
bool, "max_checkpoint_module_num": int, "selective_offload": {...}}``. Modules that are sharding
units are recomputed by the sharded engine itself; others get their ``forward`` replaced by a
checkpointed call. ``selective_offload`` moves chosen saved activations to pinned host memory on a
copy stream instead of recomputing them.
(Reference: atorch/auto/opt_lib/checkpoint_optimization.py:15-271,
selective_offloading_checkpoint.py:68-252.)
"""
from __future__ import annotations

import functools

import torch

from ...utils.checkpoint import checkpoint_function
from .optimization import Optimization


def _norm(config):
    if isinstance(config, dict):
        cfg = dict(config)
    else:
        cfg = {"wrap_class": config}
    wc = cfg.get("wrap_class", ())
    if wc is None:
        wc = ()
    if not isinstance(wc, (tuple, list, set)):
        wc = (wc,)
    cfg["wrap_class"] = tuple(wc)
    return cfg


def _matches(m, classes) -> bool:
    for c in classes:
        if isinstance(c, str):
            if type(m).__name__ == c:
                return True
        elif isinstance(m, c):
            return True
    return False


def apply_checkpoint(model, cfg) -> int:
    cfg = _norm(cfg)
    limit = cfg.get("max_checkpoint_module_num", -1)
    count = 0
    offload = cfg.get("selective_offload")
    for m in model.modules():
        if not _matches(m, cfg["wrap_class"]):
            continue
        if 0 <= limit <= count:
            break
        unit = getattr(m, "_atb_fsdp_unit", None)
        if unit is not None and not offload:
            unit.checkpoint = True
            count += 1
            continue
        if getattr(m, "_atb_checkpointed", False):
            continue
        inner = m.forward
        if offload:
            from ...utils.selective_offload import offload_forward

            m.forward = offload_forward(inner, offload)
        else:
            @functools.wraps(inner)
            def fwd(*a, _inner=inner, **k):
                if not torch.is_grad_enabled():
                    return _inner(*a, **k)
                return checkpoint_function(_inner, *a, preserve_rng_state=True, **k)
            m.forward = fwd
        m._atb_checkpointed = True
        count += 1
    return count


def _checkpoint_wrapper(model_context, wrapper_name, wrapper_config=None):
    apply_checkpoint(model_context.model, wrapper_config)
    return model_context


class CheckpointOptimization(Optimization):
    def __init__(self):
        super().__init__("checkpoint", "checkpoint", False)

    def transform(self, model_context, config=None):
        model_context.add_wrapper("checkpoint", _checkpoint_wrapper, _norm(config), is_pre_wrapper=True)
        return model_context
