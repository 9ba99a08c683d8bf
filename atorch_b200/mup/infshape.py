"""Shapes with a memory of the base model: every dimension of a parameter carries the size it has in the base model,
and a dimension whose size differs from its base size is a *width* ("infinite") dimension.

``InfDim(base_dim, dim)``  one dimension; ``width_mult() = dim / base_dim`` for a width dimension, 1 otherwise.
``InfShape([...])``        a tuple of them, attached to a parameter as ``p.infshape``. ``main`` is the last width
                           dimension (fan-in for a hidden matrix ``[out, in]``), and ``width_mult()`` is its multiplier.
(Reference: atorch/mup/infshape.py:9-139.)
"""
from __future__ import annotations

import copy
from typing import Iterable, List, Optional


class InfDim:
    __slots__ = ("base_dim", "dim")

    def __init__(self, base_dim: Optional[int], dim: Optional[int]):
        self.base_dim, self.dim = base_dim, dim

    def isinf(self) -> bool:
        return self.base_dim is not None and self.base_dim != self.dim

    def width_mult(self):
        return self.dim / self.base_dim if self.isinf() else 1

    def __eq__(self, other) -> bool:
        return isinstance(other, InfDim) and (self.base_dim, self.dim) == (other.base_dim, other.dim)

    def __hash__(self):
        return hash((self.base_dim, self.dim))

    def __repr__(self) -> str:
        return f"InfDim({self.base_dim}, {self.dim})"

    def __str__(self) -> str:
        return repr(self) if self.isinf() else f"FinDim({self.dim})"


class InfShape(tuple):
    def __new__(cls, dims: Iterable[InfDim] = ()):
        dims = tuple(dims)
        if not all(isinstance(d, InfDim) for d in dims):
            raise ValueError("Elements of InfShape needs to be of class InfDim")
        self = super().__new__(cls, dims)
        self.main_idx = self.main = None
        for i in range(len(dims) - 1, -1, -1):
            if dims[i].isinf():
                self.main_idx, self.main = i, dims[i]
                break
        return self

    def ninf(self) -> int:
        return sum(d.isinf() for d in self)

    def width_mult(self):
        return self.main.width_mult() if self.main is not None else 1

    def fanin_fanout(self):
        assert len(self) >= 2, "fanin, fanout undefined for 1-dimensional weights"
        return self[1], self[0]

    def fanin_fanout_mult_ratio(self):
        fan_in, fan_out = self.fanin_fanout()
        return fan_in.width_mult() / fan_out.width_mult()

    def base_shape(self) -> List[Optional[int]]:
        return [d.base_dim for d in self]

    def shape(self) -> List[Optional[int]]:
        return [d.dim for d in self]

    def serialize(self) -> dict:
        return {"base_shape": self.base_shape(), "shape": self.shape()}

    @classmethod
    def deserialize(cls, d: dict) -> "InfShape":
        return cls(InfDim(b, s) for b, s in zip(d["base_shape"], d["shape"]))

    @classmethod
    def from_base_shape(cls, base_shape) -> "InfShape":
        return cls(InfDim(b, None) for b in base_shape)

    def __eq__(self, other) -> bool:
        return isinstance(other, InfShape) and len(self) == len(other) and all(a == b for a, b in zip(self, other))

    def __hash__(self):
        return tuple.__hash__(self)

    def __deepcopy__(self, memo):
        return InfShape(copy.copy(d) for d in self)

    def __repr__(self) -> str:
        return "InfShape([" + ", ".join(repr(d) for d in self) + "])"


def zip_infshape(base_dims, dims, fin_if_same: bool = True) -> InfShape:
    """Pair base sizes (ints, or ``InfDim``s whose ``base_dim`` is kept) with actual sizes. An int base size equal to
    the actual size gives a finite dimension unless ``fin_if_same`` is off."""
    out = []
    for b, d in zip(base_dims, dims):
        if isinstance(b, InfDim):
            out.append(InfDim(b.base_dim, d))
        elif isinstance(b, int):
            out.append(InfDim(None if (b == d and fin_if_same) else b, d))
        else:
            raise ValueError(f"unhandled base_dim type: {type(b)}")
    return InfShape(out)
