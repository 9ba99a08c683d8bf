"""Building models that do not fit in host memory: meta-device construction with values bound later.

* ``init_empty_weights_with_disk_offload(ckpt_path=..., shard_kwargs=...)``: context under which
  modules are built with parameters on the meta device; if a flat checkpoint path is given the model
  is bound to it, so the sharded engine fills each rank's shard straight from the checkpoint.
* ``record_module_init`` / ``build_recorded_module``: remember constructor arguments so a module can
  be rebuilt (on another device, or sharded) later.
* ``reload_meta_module`` / ``materialize_modules_to_device``: give real storage to what is still meta.
(Reference: atorch/utils/meta_model_utils.py:56-895.)
"""
from __future__ import annotations

import contextlib
import functools
from typing import Callable, Dict, Optional

import torch
import torch.nn as nn

_BOUND_CKPT: Dict[int, dict] = {}


@contextlib.contextmanager
def init_empty_weights_with_disk_offload(ignore_tie_weights: bool = False, include_buffers: bool = False,
                                         disk_offload: bool = False, checkpoint_name: Optional[str] = None,
                                         ckpt_path: Optional[str] = None, shard_kwargs: Optional[dict] = None, **_):
    """Parameters created inside live on the meta device. With ``ckpt_path`` the resulting model
    (see ``bind_checkpoint``) is filled from that flat checkpoint when it is sharded."""
    reg = nn.Module.register_parameter
    state = {"ckpt_path": ckpt_path, "shard_kwargs": shard_kwargs or {}, "modules": []}

    def register_parameter(module, name, param):
        reg(module, name, param)
        if param is not None and not param.is_meta:
            cls = type(module._parameters[name])
            kw = module._parameters[name].__dict__
            module._parameters[name] = cls(module._parameters[name].to("meta"), requires_grad=param.requires_grad)
            module._parameters[name].__dict__.update(kw)
        if ckpt_path is not None:
            module._atb_ckpt_binding = state

    nn.Module.register_parameter = register_parameter
    try:
        with torch.device("meta") if include_buffers else contextlib.nullcontext():
            yield state
    finally:
        nn.Module.register_parameter = reg


def bound_checkpoint(model: nn.Module) -> Optional[dict]:
    for m in model.modules():
        b = getattr(m, "_atb_ckpt_binding", None)
        if b is not None and b.get("ckpt_path"):
            return b
    return None


def is_meta(module: nn.Module) -> bool:
    return any(p.is_meta for p in module.parameters()) or any(b.is_meta for b in module.buffers())


def record_module_init():
    """Make every ``nn.Module`` built from now on remember its constructor arguments
    (``module._init_args``); returns an undo function: ``undo = record_module_init(); build(); undo()``."""
    def __new__(cls, *a, **k):
        obj = object.__new__(cls)
        object.__setattr__(obj, "_init_args", (a, k))
        return obj
    nn.Module.__new__ = __new__

    def undo():
        # a plain pass-through stays in place: deleting a once-set __new__ leaves CPython rejecting
        # constructor arguments in object.__new__
        def plain_new(cls, *a, **k):
            return object.__new__(cls)
        nn.Module.__new__ = plain_new
    return undo


def build_recorded_module(module: nn.Module, device=None) -> nn.Module:
    """Re-run the recorded constructor of ``module`` (optionally under a device context)."""
    if not hasattr(module, "_init_args"):
        raise ValueError("module was not built under record_module_init()")
    a, k = module._init_args
    with (torch.device(device) if device is not None else contextlib.nullcontext()):
        return type(module)(*a, **k)


def materialize_modules_to_device(module: nn.Module, device, init_fn: Optional[Callable] = None) -> nn.Module:
    for m in module.modules():
        if any(p.is_meta for p in m._parameters.values() if p is not None) or \
                any(b.is_meta for b in m._buffers.values() if b is not None):
            m.to_empty(device=device, recurse=False)
            if init_fn is not None:
                init_fn(m)
            elif hasattr(m, "reset_parameters"):
                m.reset_parameters()
    return module.to(device)


def reload_meta_module(module: nn.Module, device="cpu", delete_ckpt_name: bool = True) -> nn.Module:
    """Give storage to parameters still on meta; values come from the bound checkpoint when there is one."""
    b = bound_checkpoint(module)
    materialize_modules_to_device(module, device)
    if b is not None:
        from .fsdp_save_util import ShardTensorUtil

        util = ShardTensorUtil(b["ckpt_path"], **{k: v for k, v in b["shard_kwargs"].items()
                                                   if k in ("name_mapping_func_or_dict",)})
        with torch.no_grad():
            for n, p in module.named_parameters():
                t = util.load_tensor_by_name(n, strict=False)
                if t is not None:
                    p.copy_(t.to(p.dtype))
    return module
