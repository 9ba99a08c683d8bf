"""``PrecisionSwitchableLinear``: one set of weights, two compute paths (bf16 and block-scaled fp8),
selectable at run time (``switch_precision("fp8" | "original")``), so that a model can warm up in
bf16 and continue in fp8 or evaluate either way. ``fp8_input_current_scaling`` is implied by the
tile-scaled recipe (scales always come from the current tensor).
(Reference: atorch/modules/fp8/precision_switchable_linear.py:26-228.)
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from .scaled_linear import ScaledLinear


class PrecisionSwitchableLinear(ScaledLinear):
    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None, selection: str = "fp8",
                 use_input_current_scaling: bool = False, **kw):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype, **kw)
        self.selection = selection
        self.use_fp8 = selection == "fp8"

    @classmethod
    def from_linear(cls, lin: nn.Linear, selection: str = "fp8", **kw):
        m = cls(lin.in_features, lin.out_features, bias=lin.bias is not None, device=lin.weight.device,
                dtype=lin.weight.dtype, selection=selection, **kw)
        m.weight = lin.weight
        if lin.bias is not None:
            m.bias = lin.bias
        return m

    def switch_precision(self, selection: str) -> None:
        assert selection in ("fp8", "original")
        self.selection, self.use_fp8 = selection, selection == "fp8"

    def get_extra_state(self):
        return {"selection": self.selection}

    def set_extra_state(self, state):
        if state:
            self.switch_precision(state.get("selection", self.selection))
