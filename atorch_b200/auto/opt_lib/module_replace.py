"""``module_replace``: swap library modules for this framework's fused ones, keeping weights and
checkpoint names.

A *pair* is ``name -> (source class, target class, kwargs, supported dtypes, need_src_module)``;
``register_replace_pair`` adds user pairs. Config ``None`` applies every registered pair that fits
the current half-precision dtype; a dict ``{pair_name: kwargs}`` applies only those.
(Reference: atorch/auto/opt_lib/module_replace_optimization.py:22-184,
atorch/modules/transformer/inject.py:131-256.)
"""
from __future__ import annotations

import logging
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from ..auto_accelerate_context import AutoAccelerateContext
from .optimization import Optimization

logger = logging.getLogger("atorch.logger")

REPLACEMENT_PAIRS: Dict[str, Tuple] = {}


def register_replace_pair(pair_name: str, kwargs: Optional[dict] = None, supported_dtypes=None, pair_cls=None) -> None:
    """``pair_cls`` = (source class, target class). The target is built as
    ``target(src_module, **kwargs)`` if it defines ``from_module`` / accepts the source module, and
    must expose the same parameter names as the source so state dicts keep loading."""
    if pair_cls is None:
        raise ValueError("pair_cls=(src_cls, target_cls) is required")
    dtypes = set(supported_dtypes) if supported_dtypes else {torch.float32, torch.float16, torch.bfloat16}
    REPLACEMENT_PAIRS[pair_name] = (pair_cls[0], pair_cls[1], dict(kwargs or {}), dtypes)


def _register_defaults() -> None:
    if REPLACEMENT_PAIRS:
        return
    from ...modules.normalization import AtorchLayerNorm
    from ...modules.transformer.layers import (BertAttentionFA, CLIPAttentionFA, GPT2AttentionFA, LlamaAttentionFA,
                                               MultiheadAttentionFA, hf_classes)

    half = {torch.float16, torch.bfloat16}
    register_replace_pair("LayerNorm_Apex", pair_cls=(nn.LayerNorm, AtorchLayerNorm))
    register_replace_pair("MultiheadAttention_FA", supported_dtypes=half,
                          pair_cls=(nn.MultiheadAttention, MultiheadAttentionFA))
    hf = hf_classes()
    for nm, src, tgt in (("HF_LlamaAttention_FA", hf.get("LlamaAttention"), LlamaAttentionFA),
                         ("HF_BertAttention_FA", hf.get("BertAttention"), BertAttentionFA),
                         ("HF_GPT2Attention_FA", hf.get("GPT2Attention"), GPT2AttentionFA),
                         ("HF_CLIPAttention_FA", hf.get("CLIPAttention"), CLIPAttentionFA)):
        if src is not None:
            register_replace_pair(nm, supported_dtypes=half, pair_cls=(src, tgt))


def _build_target(src: nn.Module, target_cls, kwargs):
    if hasattr(target_cls, "from_module"):
        return target_cls.from_module(src, **kwargs)
    return target_cls(src, **kwargs)


def replace_module(model: nn.Module, src_cls, target_cls, kwargs: Optional[dict] = None) -> int:
    """Replace every ``src_cls`` instance (exact type) below ``model``; returns the count."""
    n = 0
    for parent in list(model.modules()):
        for name, child in list(parent._modules.items()):
            if child is not None and type(child) is src_cls:
                parent._modules[name] = _build_target(child, target_cls, kwargs or {})
                n += 1
    return n


def _module_replace_wrapper(model_context, wrapper_name, wrapper_config=None):
    _register_defaults()
    dtype = AutoAccelerateContext.get("half_precision_dtype", torch.float32)
    cfg = wrapper_config
    verbose = False
    if isinstance(cfg, dict):
        cfg = dict(cfg)
        verbose = bool(cfg.pop("verbose", False))
    names = list(REPLACEMENT_PAIRS) if not cfg else list(cfg)
    for pn in names:
        if pn not in REPLACEMENT_PAIRS:
            logger.warning("module_replace: unknown pair %s", pn)
            continue
        src, tgt, kwargs, dtypes = REPLACEMENT_PAIRS[pn]
        if dtype not in dtypes:
            continue
        kw = dict(kwargs)
        if cfg and isinstance(cfg.get(pn), dict):
            kw.update(cfg[pn])
        n = replace_module(model_context.model, src, tgt, kw)
        if verbose and n:
            logger.info("module_replace: %s replaced %d modules", pn, n)
    return model_context


class ModuleReplaceOptimization(Optimization):
    def __init__(self):
        super().__init__("module_replace", "module_replace", False)

    def transform(self, model_context, config=None):
        model_context.add_wrapper("module_replace", _module_replace_wrapper, config, is_pre_wrapper=True)
        return model_context
