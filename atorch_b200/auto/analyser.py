"""Static facts about a model used by the search: parameter counts, sizes, dominant repeated block
class (the natural sharding / checkpoint unit), replaceable modules, forward FLOPs of linear layers.
(Reference: atorch/auto/analyser/analyser.py:14.)
"""
from __future__ import annotations

from collections import Counter
from typing import Dict

import torch.nn as nn


def analyse_model(model: nn.Module) -> Dict:
    total = sum(p.numel() for p in model.parameters())
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    nbytes = sum(p.numel() * p.element_size() for p in model.parameters())
    cls_params: Counter = Counter()
    cls_count: Counter = Counter()
    for m in model.modules():
        if m is model:
            continue
        n = sum(p.numel() for p in m.parameters())
        if n:
            cls_params[type(m)] += n
            cls_count[type(m)] += 1
    # the repeated block: a class appearing several times that owns the largest share of parameters;
    # composite modules (with children) win over leaf layers such as nn.Linear
    has_children = {type(m) for m in model.modules() if len(m._modules) > 0}
    block = None
    for composite in (True, False):
        best = 0
        for c, cnt in cls_count.items():
            if cnt < 2 or issubclass(c, (nn.ModuleList, nn.Sequential, nn.ModuleDict)):
                continue
            if (c in has_children) != composite:
                continue
            if cls_params[c] > best:
                block, best = c, cls_params[c]
        if block is not None:
            break
    linear_flops = sum(2 * m.in_features * m.out_features for m in model.modules() if isinstance(m, nn.Linear))
    from .opt_lib.module_replace import REPLACEMENT_PAIRS, _register_defaults

    try:
        _register_defaults()
    except Exception:
        pass
    replaceable = [n for n, (src, *_r) in REPLACEMENT_PAIRS.items() if any(type(m) is src for m in model.modules())]
    return {"model_params_num": total, "model_params_mb": nbytes / 2 ** 20, "trainable_params_num": trainable,
            "opt_config_submodule_names": (block,) if block is not None else (),
            "submodule_types": {c.__name__: n for c, n in cls_count.items()},
            "linear_flops_per_sample_row": linear_flops, "replaceable_pairs": replaceable}
