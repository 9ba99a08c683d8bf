"""Initialising a sharded model from a flat checkpoint.

``FSDPCkptConfig`` names the checkpoint (and LoRA extras); ``FSDPInitFn`` is a ``param_init_fn`` for the
``fsdp`` optimisation: every rank materialises a module on its device and fills the parameters it can
find in the checkpoint directly from the shard files (byte-range reads, any saved world size);
parameters missing from the checkpoint keep their fresh initialisation. No rank-0 load + broadcast.
(Reference: atorch/utils/fsdp_init_util.py:45-683, which swaps torch FSDP's FlatParamHandle.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Optional

import torch
import torch.nn as nn

from .fsdp_save_util import ShardTensorUtil


@dataclass
class FSDPCkptConfig:
    flat_ckpt_path: Optional[str] = None
    lora_ckpt_path: Optional[str] = None
    lora_prefix: Optional[str] = None
    lora_cls: Optional[tuple] = None
    lora_weight_name: Optional[str] = None
    name_mapping: Optional[Dict[str, str]] = None


class FSDPInitFn:
    def __init__(self, top_model: nn.Module, rank: int, ckpt_config: FSDPCkptConfig,
                 post_init_fn: Optional[Callable[[nn.Module], None]] = None, device=None):
        self.rank, self.cfg, self.post_init_fn = rank, ckpt_config, post_init_fn
        self.device = device
        self.names = {id(m): n for n, m in top_model.named_modules()}
        self.util = ShardTensorUtil(ckpt_config.flat_ckpt_path, rank, 1, "cpu", ckpt_config.name_mapping) \
            if ckpt_config.flat_ckpt_path else None
        self.loaded, self.missing = [], []

    def __call__(self, module: nn.Module) -> None:
        if hasattr(module, "reset_parameters"):
            module.reset_parameters()
        prefix = self.names.get(id(module), "")
        with torch.no_grad():
            for n, p in module._parameters.items():
                if p is None:
                    continue
                fqn = f"{prefix}.{n}" if prefix else n
                t = self.util.load_tensor_by_name(fqn, strict=False) if self.util is not None else None
                if t is not None:
                    p.copy_(t.to(device=p.device, dtype=p.dtype))
                    self.loaded.append(fqn)
                else:
                    self.missing.append(fqn)
        if self.post_init_fn is not None:
            self.post_init_fn(module)
