"""Optimizers with muP learning-rate scaling, as a rewrite of the parameter groups handed to any optimizer class.

Adam-like optimizers (entrywise-normalised updates): a hidden matrix (two width dimensions) gets ``lr / width_mult``
and, with ``scaled_wd``, ``weight_decay * width_mult``; everything else keeps the group's values.
SGD-like optimizers: a vector-like parameter (one width dimension) gets ``lr * width_mult`` and
``weight_decay / width_mult``; a hidden matrix ``lr / r`` and (``scaled_wd``) ``weight_decay * r`` with
``r = fan-in multiplier / fan-out multiplier``; parameters without width dimensions are untouched.
``MuAdam(params, impl=AdamW, ...)`` / ``MuSGD(params, impl=SGD, ...)`` build the optimizer; the ``*ParamGroupsAdjust``
functions return the groups only.
(Reference: atorch/mup/optim.py:30-133.)
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, List

from torch.optim import SGD, AdamW


def process_param_groups(params, **kwargs) -> List[dict]:
    """A list of group dicts, each with its own ``lr`` and ``weight_decay`` filled in from the keyword defaults."""
    groups = list(params)
    if groups and not isinstance(groups[0], dict):
        groups = [{"params": groups}]
    for g in groups:
        if "lr" not in g:
            g["lr"] = kwargs["lr"]
        g.setdefault("weight_decay", kwargs.get("weight_decay", 0.0))
    return groups


def _infshape_of(p, do_assert: bool):
    shp = getattr(p, "infshape", None)
    if do_assert:
        assert shp is not None, (f"A parameter with shape {tuple(p.shape)} does not have `infshape` attribute. "
                                 "Did you forget to call `mup.set_base_shapes` on the model?")
    if shp is not None and shp.ninf() > 2:
        raise NotImplementedError("more than 2 inf dimensions")
    return shp


def _split(group: dict, classify: Callable) -> "OrderedDict":
    """Parameters of one group bucketed by ``classify(p) -> hashable key``; each bucket inherits the group's options."""
    buckets: "OrderedDict" = OrderedDict()
    for p in group["params"]:
        key = classify(p)
        if key not in buckets:
            buckets[key] = dict({k: v for k, v in group.items() if k != "params"}, params=[])
        buckets[key]["params"].append(p)
    return buckets


def MuAdamParamGroupsAdjust(params, scaled_wd: bool = True, do_assert: bool = True, **kwargs) -> List[dict]:
    out = []
    for group in process_param_groups(params, **kwargs):
        def classify(p):
            shp = _infshape_of(p, do_assert)
            return ("matrix", shp.width_mult()) if shp is not None and shp.ninf() == 2 else ("vector", 1)

        buckets = _split(group, classify)
        vector = buckets.pop(("vector", 1), dict({k: v for k, v in group.items() if k != "params"}, params=[]))
        for (_, mult), g in buckets.items():
            g["lr"] /= mult
            if scaled_wd:
                g["weight_decay"] *= mult
            out.append(g)
        out.append(vector)
    return out


def MuSGDParamGroupsAdjust(params, scaled_wd: bool = True, do_assert: bool = True, **kwargs) -> List[dict]:
    out = []
    for group in process_param_groups(params, **kwargs):
        def classify(p):
            shp = _infshape_of(p, do_assert)
            if shp is None or shp.ninf() == 0:
                return ("fixed", 1)
            return ("vector", shp.width_mult()) if shp.ninf() == 1 else ("matrix", shp.fanin_fanout_mult_ratio())

        buckets = _split(group, classify)
        fixed = buckets.pop(("fixed", 1), dict({k: v for k, v in group.items() if k != "params"}, params=[]))
        matrices = [(k, g) for k, g in buckets.items() if k[0] == "matrix"]
        vectors = [(k, g) for k, g in buckets.items() if k[0] == "vector"]
        for (_, ratio), g in matrices:
            g["lr"] /= ratio
            if scaled_wd:
                g["weight_decay"] *= ratio
            out.append(g)
        for (_, mult), g in vectors:
            g["lr"] *= mult
            g["weight_decay"] /= mult
            out.append(g)
        out.append(fixed)
    return out


def MuAdam(params, impl=AdamW, scaled_wd: bool = True, do_assert: bool = True, **kwargs):
    """``impl`` over the muP-adjusted groups. The model's base shapes must have been set (``set_base_shapes``)."""
    return impl(MuAdamParamGroupsAdjust(params, scaled_wd=scaled_wd, do_assert=do_assert, **kwargs), **kwargs)


def MuSGD(params, impl=SGD, scaled_wd: bool = True, do_assert: bool = True, **kwargs):
    return impl(MuSGDParamGroupsAdjust(params, scaled_wd=scaled_wd, do_assert=do_assert, **kwargs), **kwargs)
