"""Base shapes: which dimensions of a model's parameters are widths, and their sizes in the base model.

``set_base_shapes(model, base, delta=None, savefile=None, do_assert=True)`` attaches ``p.infshape`` to every parameter
of ``model``. ``base`` is a module, a dict of shapes / ``InfShape``s, the path of a base-shape file (yaml: parameter
name -> list of base sizes, ``null`` for a non-width dimension once made from a base/delta pair) or ``None`` (the model
is its own base). With a ``delta`` model, exactly the dimensions that differ between base and delta are widths, so a
target that equals the base in some width still knows it; without one, a dimension is a width where target and base
differ. Readout layers get their width multiplier set at the end.
(Reference: atorch/mup/shape.py:20-228.)
"""
from __future__ import annotations

import copy
from typing import Dict, Union

import yaml
from torch import nn

from .infshape import InfShape, zip_infshape

_FILE_HEADER = ("# base shapes (yaml): parameter name -> its sizes in the base model\n"
                "# a number is the base size of a width dimension, null marks a dimension that does not scale\n")


def get_shapes(model) -> dict:
    """Parameter shapes by name; a model may supply its own ``get_shapes()``."""
    if hasattr(model, "get_shapes"):
        return model.get_shapes()
    return {n: p.shape for n, p in model.named_parameters()}


def get_infshapes(model) -> Dict[str, InfShape]:
    return {n: p.infshape for n, p in model.named_parameters()}


def load_base_shapes(filename: str) -> Dict[str, InfShape]:
    with open(filename) as f:
        return {k: InfShape.from_base_shape(v) for k, v in yaml.safe_load(f).items()}


def _shapes_of(x) -> dict:
    if isinstance(x, nn.Module):
        return get_shapes(x)
    if isinstance(x, dict):
        return copy.deepcopy(x)
    if isinstance(x, str):
        return load_base_shapes(x)
    raise ValueError(f"unhandled x type: {type(x)}")


def save_base_shapes(model_or_shapes: Union[nn.Module, dict], file) -> None:
    if isinstance(model_or_shapes, nn.Module):
        table = {k: list(s) for k, s in get_shapes(model_or_shapes).items()}
    elif isinstance(model_or_shapes, dict):
        table = {k: (s.base_shape() if isinstance(s, InfShape) else list(s)) for k, s in model_or_shapes.items()}
    else:
        raise ValueError(f"unhandled type: {type(model_or_shapes)}")
    if file:
        with open(file, "w") as f:
            f.write(_FILE_HEADER + yaml.dump(table, None, indent=4))


def _align_wrapper_prefix(base: dict, target: dict):
    """A (Distributed)DataParallel wrapper prefixes every name with ``module.``: give the base names the target's form."""
    pre = "module."
    if all(k.startswith(pre) for k in target) and not any(k.startswith(pre) for k in base):
        base = {pre + k: v for k, v in base.items()}
    elif not any(k.startswith(pre) for k in target) and base and all(k.startswith(pre) for k in base):
        base = {k[len(pre):]: v for k, v in base.items()}
    return base


def _zip_dicts(base: dict, target: dict) -> Dict[str, InfShape]:
    base = _align_wrapper_prefix(base, target)
    extra, missing = set(base) - set(target), set(target) - set(base)
    assert not extra and not missing, f"`base_shapes` has extra names {extra}. `shapes` has extra names {missing}."
    return {name: zip_infshape(b, target[name]) for name, b in base.items()}


def zip_infshapes(base, target) -> Dict[str, InfShape]:
    return _zip_dicts(_shapes_of(base), _shapes_of(target))


def clear_dims(infshapes: Dict[str, InfShape]) -> Dict[str, InfShape]:
    """The same table with every actual size forgotten (only base sizes and the width marks remain)."""
    return {k: InfShape.from_base_shape(v.base_shape()) for k, v in infshapes.items()}


def make_base_shapes(base_shapes, delta_shapes, savefile=None) -> Dict[str, InfShape]:
    """The base-shape table of a (base, delta) pair: dimensions that differ are widths with the base's size."""
    table = clear_dims(zip_infshapes(base_shapes, delta_shapes))
    if savefile is not None:
        save_base_shapes(table, savefile)
    return table


def apply_infshapes(model: nn.Module, infshapes: Dict[str, InfShape]) -> None:
    for name, p in model.named_parameters():
        p.infshape = infshapes[name]


def assert_hidden_size_inf(model: nn.Module) -> None:
    """A plain linear layer that maps a width dimension to a fixed one must be an ``OutputLayer``."""
    from .module import OutputLayer

    for name, m in model.named_modules():
        if isinstance(m, nn.Linear) and not isinstance(m, OutputLayer):
            shp = m.weight.infshape
            assert shp[0].isinf() or not shp[1].isinf(), (
                f"{name} has infinite fan-in and finite fan-out dimensions but is not type `OutputLayer`. "
                "To resolve this, either change the module to `OutputLayer` or change the fan-out to an infinite "
                "dimension.")


def set_base_shapes(model: nn.Module, base, delta=None, savefile=None, do_assert: bool = True) -> nn.Module:
    from .module import OutputLayer

    base_shapes = _shapes_of(model if base is None else base)
    if delta is not None:
        base_shapes = _zip_dicts(base_shapes, _shapes_of(delta))
    infshapes = _zip_dicts(base_shapes, get_shapes(model))
    if savefile is not None:
        save_base_shapes(infshapes, savefile)
    apply_infshapes(model, infshapes)
    if do_assert:
        assert_hidden_size_inf(model)
    for m in model.modules():
        if isinstance(m, OutputLayer):
            m.set_width_mult()
    return model
