"""Maximal update parametrisation (muP): hyper-parameters tuned on a narrow model carry over to wide ones.

1. build the model from ``MupLinear`` / ``QKVLayer`` / ``QLayer`` / ``OutputLayer`` (``module.py``);
2. ``set_base_shapes(model, base, delta)`` marks the width dimensions of every parameter (``shape.py``,
   ``infshape.py``; base shapes can be saved to and loaded from a yaml file);
3. ``model.mup_initial("mup")`` draws width-aware initial weights (``init.py`` has the drop-in initialisers);
4. ``MuAdam`` / ``MuSGD`` scale per-parameter learning rates and weight decay (``optim.py``).
(Reference: atorch/mup/{infshape,shape,init,module,optim}.py.)
"""
from .infshape import InfDim, InfShape, zip_infshape
from .module import MupLinear, MupModule, OutputLayer, QKVLayer, QLayer, SharedOutputLayer
from .optim import MuAdam, MuAdamParamGroupsAdjust, MuSGD, MuSGDParamGroupsAdjust, process_param_groups
from .shape import (apply_infshapes, assert_hidden_size_inf, clear_dims, get_infshapes, get_shapes, load_base_shapes,
                    make_base_shapes, save_base_shapes, set_base_shapes, zip_infshapes)

__all__ = ["InfDim", "InfShape", "zip_infshape", "MupLinear", "MupModule", "OutputLayer", "QKVLayer", "QLayer",
           "SharedOutputLayer", "MuAdam", "MuAdamParamGroupsAdjust", "MuSGD", "MuSGDParamGroupsAdjust",
           "process_param_groups", "apply_infshapes", "assert_hidden_size_inf", "clear_dims", "get_infshapes",
           "get_shapes", "load_base_shapes", "make_base_shapes", "save_base_shapes", "set_base_shapes", "zip_infshapes"]
