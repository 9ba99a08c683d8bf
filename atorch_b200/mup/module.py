"""Linear layers that know how to initialise themselves under muP or under the standard parametrisation (SP).

Nothing happens at construction: ``mup_initial(mode)`` (on a layer, or on a ``MupModule`` for all layers below it)
draws the weights. ``sampler`` names the distribution (``uniform``, ``normal``, ``xavier_uniform``, ``xavier_normal``,
``kaiming_uniform``, ``kaiming_normal``; its arguments come as keyword arguments of the layer); under ``"mup"`` the
width-aware initialisers are used, under ``"sp"`` torch's. ``init_weight_method`` / ``init_bias_method`` override both.

``QKVLayer`` / ``QLayer``   zero the query rows (attention logits start at zero).
``OutputLayer``             the readout: forward computes ``linear(output_mult * x / width_mult)``; under muP its SP
                            draw is scaled by ``width_mult ** 0.5`` (or zeroed with ``weight_zero_init``).
``SharedOutputLayer``       a readout tied to an embedding weight.
(Reference: atorch/mup/module.py:11-303.)
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch import nn

from . import init as mup_init

_SAMPLERS = {          # sampler name -> (keyword defaults, muP initialiser, torch initialiser)
    "uniform": (dict(a=0.0, b=1.0), mup_init.uniform_, nn.init.uniform_),
    "normal": (dict(mean=0.0, std=1.0), mup_init.normal_, nn.init.normal_),
    "xavier_uniform": (dict(gain=1.0), mup_init.xavier_uniform_, nn.init.xavier_uniform_),
    "xavier_normal": (dict(gain=1.0), mup_init.xavier_normal_, nn.init.xavier_normal_),
    "kaiming_uniform": (dict(a=0.0, mode="fan_in", nonlinearity="leaky_relu"), mup_init.kaiming_uniform_,
                        nn.init.kaiming_uniform_),
    "kaiming_normal": (dict(a=0.0, mode="fan_in", nonlinearity="leaky_relu"), mup_init.kaiming_normal_,
                       nn.init.kaiming_normal_),
}


class MupModule(nn.Module):
    """``mup_initial("mup" | "sp")`` initialises every ``MupLinear`` in the module tree."""

    def mup_initial(self, mode: str = "mup") -> None:
        assert mode in ("mup", "sp")
        self._mode = mode
        for m in self.modules():
            if isinstance(m, MupLinear):
                m.mup_initial(mode)


class MupLinear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, sampler: str = "normal",
                 bias_zero_init: bool = True, init_weight_method: Optional[Callable] = None,
                 init_bias_method: Optional[Callable] = None, device=None, dtype=None, **kwargs) -> None:
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        assert sampler in _SAMPLERS, sampler
        self._sampler, self._kwargs = sampler, kwargs
        self._bias_zero_init = bias_zero_init
        self._init_weight_method, self._init_bias_method = init_weight_method, init_bias_method

    def _draw(self, mup: bool) -> None:
        defaults, mup_fn, sp_fn = _SAMPLERS[self._sampler]
        args = {k: self._kwargs.get(k, v) for k, v in defaults.items()}
        (mup_fn if mup else sp_fn)(self.weight, **args)

    def _mup_init_weight(self) -> None:
        assert hasattr(self.weight, "infshape"), "Please call set_base_shapes(...) on the model first"
        self._draw(True)

    def _sp_init_weight(self) -> None:
        self._draw(False)

    def _mup_init_bias(self) -> None:
        with torch.no_grad():
            self.bias.mul_(self.weight.infshape[1].width_mult() ** 0.5)

    def mup_initial(self, mode: str = "mup") -> None:
        assert mode in ("mup", "sp")
        if self._init_weight_method:
            self._init_weight_method(self.weight)
        elif mode == "mup":
            self._mup_init_weight()
        else:
            self._sp_init_weight()
        if self.bias is None:
            return
        if self._init_bias_method:
            self._init_bias_method(self.bias)
        elif self._bias_zero_init:
            with torch.no_grad():
                self.bias.zero_()
        elif mode == "mup":
            self._mup_init_bias()


class QKVLayer(MupLinear):
    """Fused q | k | v projection (three equal row blocks); ``q_zero_init`` zeroes the q block in both modes."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, sampler: str = "normal",
                 q_zero_init: bool = True, bias_zero_init: bool = True, init_weight_method=None, init_bias_method=None,
                 device=None, dtype=None, **kwargs) -> None:
        super().__init__(in_features, out_features, bias, sampler, bias_zero_init, init_weight_method, init_bias_method,
                         device, dtype, **kwargs)
        self._q_zero_init = q_zero_init

    def _zero_query(self) -> None:
        if self._q_zero_init:
            rows = self.weight.shape[0]
            assert rows % 3 == 0, "a fused q/k/v weight has 3 equal row blocks"
            with torch.no_grad():
                self.weight[: rows // 3].zero_()

    def _mup_init_weight(self) -> None:
        MupLinear._mup_init_weight(self)
        self._zero_query()

    def _sp_init_weight(self) -> None:
        MupLinear._sp_init_weight(self)
        self._zero_query()


class QLayer(QKVLayer):
    """A separate query projection: the whole weight is the query block."""

    def _zero_query(self) -> None:
        if self._q_zero_init:
            with torch.no_grad():
                self.weight.zero_()


class OutputLayer(MupLinear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, output_mult: float = 1.0,
                 sampler: str = "normal", weight_zero_init: bool = False, bias_zero_init: bool = True,
                 init_weight_method=None, init_bias_method=None, device=None, dtype=None, **kwargs) -> None:
        super().__init__(in_features, out_features, bias, sampler, bias_zero_init, init_weight_method, init_bias_method,
                         device, dtype, **kwargs)
        self._output_mult, self._weight_zero_init, self._width_mult = output_mult, weight_zero_init, 1.0

    output_mult = property(lambda self: self._output_mult)

    def set_width_mult(self) -> None:
        """Called by ``set_base_shapes``: the multiplier of the weight's (only) width dimension."""
        self._width_mult = self.weight.infshape.width_mult()

    def width_mult(self) -> float:
        return self._width_mult

    def _mup_init_weight(self) -> None:
        self._draw(False)                        # the SP draw, then the muP correction
        with torch.no_grad():
            if self._weight_zero_init:
                self.weight.zero_()
            else:
                self.weight.mul_(self._width_mult ** 0.5)

    def _sp_init_weight(self) -> None:
        self._draw(False)
        if self._weight_zero_init:
            with torch.no_grad():
                self.weight.zero_()

    def _mup_init_bias(self) -> None:
        with torch.no_grad():
            self.bias.mul_(self._width_mult ** 0.5)

    def forward(self, x):
        return super().forward(self._output_mult * x / self._width_mult)


class SharedOutputLayer(OutputLayer):
    """``weight`` is the ``[vocab, width]`` weight of an ``nn.Embedding``; the other arguments as for ``OutputLayer``."""

    def __init__(self, weight: nn.Parameter, bias: bool = True, **kwargs):
        super().__init__(weight.shape[1], weight.shape[0], bias=bias, **kwargs)
        self.weight = weight
