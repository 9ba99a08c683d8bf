"""Maximal update parametrisation (muP): width-aware initialisation, output scaling and optimizers
so that hyper-parameters tuned on a narrow model transfer to wide ones.

``set_base_shapes(model, base, delta)`` attaches an ``InfShape`` to every parameter (which dims grow
with width, and by how much relative to the base model); ``MupLinear`` / ``OutputLayer`` apply the
forward multipliers; ``MuAdam`` / ``MuSGD`` rescale per-parameter learning rates and weight decay.
(Reference: atorch/mup/{shape.py:170-204, infshape.py:9-120, module.py:29-302, optim.py:42-133, init.py}.)
"""
from __future__ import annotations

import math
from collections import defaultdict
from typing import Optional

import torch
import torch.nn as nn


class InfDim:
    def __init__(self, base_dim: Optional[int], dim: int):
        self.base_dim, self.dim = base_dim, dim

    def isinf(self) -> bool:
        return self.base_dim is not None

    def width_mult(self) -> float:
        return self.dim / self.base_dim if self.isinf() else 1.0


class InfShape(tuple):
    def __new__(cls, dims):
        return super().__new__(cls, dims)

    def ninf(self) -> int:
        return sum(d.isinf() for d in self)

    def width_mult(self) -> float:
        if self.ninf() == 0:
            return 1.0
        if self.ninf() == 1:
            return next(d.width_mult() for d in self if d.isinf())
        return self[1].width_mult() if self[1].isinf() else self[0].width_mult()   # fan-in of a matrix [out, in]

    def fanin_fanout_mult_ratio(self) -> float:
        assert self.ninf() == 2
        return self[1].width_mult() / self[0].width_mult()


def set_base_shapes(model: nn.Module, base: Optional[nn.Module], delta: Optional[nn.Module] = None) -> nn.Module:
    """Dims that differ between ``base`` and ``delta`` (or between ``base`` and ``model``) are "infinite"
    (width) dims; with ``base=None`` the model is its own base (all multipliers 1)."""
    base_shapes = {n: p.shape for n, p in (base or model).named_parameters()}
    delta_shapes = {n: p.shape for n, p in (delta or model).named_parameters()}
    for n, p in model.named_parameters():
        bs, ds = base_shapes[n], delta_shapes[n]
        p.infshape = InfShape([InfDim(b if b != d or (base is not None and b != s) else None, s)
                               for b, d, s in zip(bs, ds, p.shape)])
    return model


class MupLinear(nn.Linear):
    """Hidden linear layer: standard forward, muP-aware ``mup_initial`` (variance 1/fan_in)."""

    def mup_initial(self, mode: str = "mup", init_std: float = 1.0):
        fan_in = self.weight.shape[1]
        nn.init.normal_(self.weight, std=init_std / math.sqrt(fan_in))
        if self.bias is not None:
            nn.init.zeros_(self.bias)


class QKVLayer(MupLinear):
    """Fused query/key/value projection (``out_features = 3 * width``, rows ordered q, k, v). With
    ``q_zero_init`` (default) the query third of the weight starts at zero, which makes the attention
    logits zero at initialisation as muP asks. (Reference: atorch/mup/module.py:148-207.)"""

    def __init__(self, *a, q_zero_init: bool = True, **k):
        super().__init__(*a, **k)
        self._q_zero_init = q_zero_init

    def mup_initial(self, mode: str = "mup", init_std: float = 1.0):
        super().mup_initial(mode, init_std)
        if self._q_zero_init:
            fan_out = self.weight.shape[0]
            assert fan_out % 3 == 0, "a fused q/k/v weight has 3 equal row blocks"
            with torch.no_grad():
                self.weight[: fan_out // 3].zero_()


class QLayer(QKVLayer):
    """Separate query projection: the whole weight starts at zero when ``q_zero_init``.
    (Reference: atorch/mup/module.py:208-219.)"""

    def mup_initial(self, mode: str = "mup", init_std: float = 1.0):
        MupLinear.mup_initial(self, mode, init_std)
        if self._q_zero_init:
            with torch.no_grad():
                self.weight.zero_()


class MupModule(nn.Module):
    """Base class whose ``mup_initial(mode)`` initialises every muP layer below it ("mup" or "sp").
    (Reference: atorch/mup/module.py:9-26.)"""

    def mup_initial(self, mode: str = "mup", init_std: float = 1.0):
        assert mode in ("mup", "sp")
        for m in self.modules():
            if m is not self and hasattr(m, "mup_initial") and not isinstance(m, MupModule):
                m.mup_initial(mode, init_std)


class OutputLayer(nn.Linear):
    """Readout layer: ``output_mult * x / width_mult`` before the matmul; zero-initialised under muP."""

    def __init__(self, *a, output_mult: float = 1.0, **k):
        super().__init__(*a, **k)
        self.output_mult = output_mult

    def width_mult(self) -> float:
        s = getattr(self.weight, "infshape", None)
        return s.width_mult() if s is not None else 1.0

    def mup_initial(self, mode: str = "mup", init_std: float = 1.0):
        if mode == "mup":
            nn.init.zeros_(self.weight)
        else:
            nn.init.normal_(self.weight, std=init_std / math.sqrt(self.weight.shape[1]))
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, x):
        return super().forward(self.output_mult * x / self.width_mult())


class SharedOutputLayer(OutputLayer):
    """Readout that shares its weight with an embedding."""

    def __init__(self, shared_weight: nn.Parameter, bias: bool = False, output_mult: float = 1.0):
        super().__init__(shared_weight.shape[1], shared_weight.shape[0], bias=bias, output_mult=output_mult)
        self.weight = shared_weight


def _split_groups(params_or_groups, defaults):
    groups = list(params_or_groups)
    if groups and not isinstance(groups[0], dict):
        groups = [{"params": groups}]
    return [dict(defaults, **g) for g in groups]


def MuAdam(params, impl=torch.optim.Adam, decoupled_wd: bool = False, **kw):
    """Adam with muP scaling: matrix-like parameters (two width dims) get ``lr / width_mult`` (and
    ``weight_decay * width_mult`` unless decoupled)."""
    out = []
    for g in _split_groups(params, kw):
        buckets = defaultdict(list)
        vector_like = []
        for p in g["params"]:
            s = getattr(p, "infshape", None)
            if s is not None and s.ninf() == 2:
                buckets[s.width_mult()].append(p)
            else:
                vector_like.append(p)
        base = {k: v for k, v in g.items() if k != "params"}
        if vector_like:
            out.append(dict(base, params=vector_like))
        for wm, ps in buckets.items():
            ng = dict(base, params=ps)
            ng["lr"] = g.get("lr", kw.get("lr", 1e-3)) / wm
            if not decoupled_wd and "weight_decay" in ng:
                ng["weight_decay"] = ng["weight_decay"] * wm
            out.append(ng)
    return impl(out, **{k: v for k, v in kw.items()})


def MuSGD(params, impl=torch.optim.SGD, decoupled_wd: bool = False, **kw):
    """SGD with muP scaling: vector-like parameters (one width dim) get ``lr * width_mult``,
    matrix-like ones ``lr / (fan_in/fan_out ratio)``."""
    out = []
    for g in _split_groups(params, kw):
        vec, mat, fixed = defaultdict(list), defaultdict(list), []
        for p in g["params"]:
            s = getattr(p, "infshape", None)
            if s is None or s.ninf() == 0:
                fixed.append(p)
            elif s.ninf() == 1:
                vec[s.width_mult()].append(p)
            else:
                mat[s.fanin_fanout_mult_ratio()].append(p)
        base = {k: v for k, v in g.items() if k != "params"}
        lr = g.get("lr", kw.get("lr", 1e-2))
        if fixed:
            out.append(dict(base, params=fixed))
        for wm, ps in vec.items():
            ng = dict(base, params=ps, lr=lr * wm)
            if not decoupled_wd and "weight_decay" in ng:
                ng["weight_decay"] = ng["weight_decay"] / wm
            out.append(ng)
        for ratio, ps in mat.items():
            ng = dict(base, params=ps, lr=lr / ratio)
            if not decoupled_wd and "weight_decay" in ng:
                ng["weight_decay"] = ng["weight_decay"] * ratio
            out.append(ng)
    return impl(out, **kw)
