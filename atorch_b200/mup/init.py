"""Width-aware counterparts of ``torch.nn.init``: identical to the torch initialisers when a tensor's shape equals
its base shape, and scaled the muP way when it is wider.

Constant-scale samplers (``uniform_``, ``normal_``, ``trunc_normal_``, ``ones_``): a hidden matrix (two width
dimensions) is drawn ``width_mult ** -0.5`` narrower, everything else unchanged; a sampler with a non-zero mean is only
allowed on tensors with exactly one width dimension. Fan-based samplers (``xavier_*``, ``kaiming_*``) undo the part of
torch's fan scaling that muP does not want. Every tensor needs the ``infshape`` that ``set_base_shapes`` attaches.
(Reference: atorch/mup/init.py:29-236.)
"""
from __future__ import annotations

import math
import warnings

import torch
from torch.nn import init as _tinit


def _infshape(t):
    assert hasattr(t, "infshape"), "Please call set_base_shapes(...)"
    return t.infshape


def _hidden_scale(t) -> float:
    n = _infshape(t).ninf()
    if n <= 1:
        return 1.0
    if n == 2:
        return t.infshape.width_mult() ** -0.5
    raise NotImplementedError("more than 2 width dimensions")


def _need_single_width(t, centred: bool) -> None:
    if not centred:
        assert _infshape(t).ninf() == 1, "Sampler for (inf, inf) tensors should have mean 0"


@torch.no_grad()
def uniform_(tensor, a=0, b=1):
    _need_single_width(tensor, a == -b)
    s = _hidden_scale(tensor)
    return tensor.uniform_(a * s, b * s)


@torch.no_grad()
def normal_(tensor, mean=0, std=1):
    _need_single_width(tensor, mean == 0)
    s = _hidden_scale(tensor)
    return tensor.normal_(mean * s, std * s)


@torch.no_grad()
def trunc_normal_(tensor, mean=0, std=1, a=-2, b=2):
    _need_single_width(tensor, mean == 0 and a == -b)
    s = _hidden_scale(tensor)
    return _tinit.trunc_normal_(tensor, mean=mean * s, std=std * s, a=a * s, b=b * s)


@torch.no_grad()
def ones_(tensor):
    _need_single_width(tensor, False)
    return tensor.fill_(_hidden_scale(tensor))


def eye_(tensor):
    _need_single_width(tensor, False)
    return _tinit.eye_(tensor)


def _xavier_std(tensor, gain: float) -> float:
    fan_in, fan_out = _tinit._calculate_fan_in_and_fan_out(tensor)
    std = gain * math.sqrt(2.0 / float(fan_in + fan_out))
    d_out, d_in = _infshape(tensor)[:2]
    base_out, base_in = d_out.base_dim or d_out.dim, d_in.base_dim or d_in.dim       # finite dims have no base size
    std *= math.sqrt((d_out.dim + d_in.dim) / (base_out + base_in))                   # back to the base model's scale
    n = tensor.infshape.ninf()
    if n == 2:
        std /= math.sqrt(d_in.width_mult())                                            # hidden matrix: like 1/fan_in
    elif n > 2:
        raise NotImplementedError("can only handle 2 inf dimensions currently")
    return std


@torch.no_grad()
def xavier_uniform_(tensor, gain=1.0):
    bound = math.sqrt(3.0) * _xavier_std(tensor, gain)
    return tensor.uniform_(-bound, bound)


@torch.no_grad()
def xavier_normal_(tensor, gain=1.0):
    return tensor.normal_(0.0, _xavier_std(tensor, gain))


def _kaiming_std(tensor, a, mode: str, nonlinearity: str) -> float:
    fan = _tinit._calculate_correct_fan(tensor, mode)
    std = _tinit.calculate_gain(nonlinearity, a) / math.sqrt(fan)
    d_out, d_in = _infshape(tensor)[:2]
    n = tensor.infshape.ninf()
    if n == 1:                         # the scale must not move with the one width dimension
        d = d_in if mode == "fan_in" else d_out
        if d.isinf():
            std *= d.width_mult() ** 0.5
    elif n == 2:                       # hidden matrix: 1/fan_in, whichever fan torch was asked for
        if mode == "fan_out":
            std *= math.sqrt(d_out.width_mult() / d_in.width_mult())
    elif n > 2:
        raise NotImplementedError("can only handle <=2 inf dimensions currently")
    return std


@torch.no_grad()
def kaiming_normal_(tensor, a=0, mode="fan_in", nonlinearity="leaky_relu"):
    if 0 in tensor.shape:
        warnings.warn("Initializing zero-element tensors is a no-op")
        return tensor
    return tensor.normal_(0, _kaiming_std(tensor, a, mode, nonlinearity))


@torch.no_grad()
def kaiming_uniform_(tensor, a=0, mode="fan_in", nonlinearity="leaky_relu"):
    if 0 in tensor.shape:
        warnings.warn("Initializing zero-element tensors is a no-op")
        return tensor
    bound = math.sqrt(3.0) * _kaiming_std(tensor, a, mode, nonlinearity)
    return tensor.uniform_(-bound, bound)
