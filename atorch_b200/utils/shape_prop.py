"""``MetaShapeProp``: run an fx graph on meta tensors and record, per node, ``meta["shape"]``,
``meta["dtype"]``, ``meta["numel"]`` and — for ``nn.Linear`` / ``nn.Embedding`` / matmul nodes — forward
``meta["flops"]``. Parameters and buffers are replaced by meta tensors for the run, so nothing is allocated
and nothing is computed. (Reference: atorch/utils/shape_prop.py.)"""
from __future__ import annotations

from typing import Any

import torch
import torch.fx as fx
import torch.nn as nn
from torch.utils._pytree import tree_map

from .tracer import meta_like


def _to_meta(x: Any) -> Any:
    return meta_like(x) if isinstance(x, torch.Tensor) and x.device.type != "meta" else x


class MetaShapeProp(fx.Interpreter):
    def __init__(self, gm: fx.GraphModule):
        super().__init__(gm, garbage_collect_values=False)

    def fetch_attr(self, target: str):
        return _to_meta(super().fetch_attr(target))

    def call_module(self, target, args, kwargs):
        m = self.fetch_submodule(target) if hasattr(self, "fetch_submodule") else self.module.get_submodule(target)
        # functional call with meta parameters: the module's own tensors stay where they are
        params = {k: meta_like(v) for k, v in list(m.named_parameters()) + list(m.named_buffers())}
        return torch.func.functional_call(m, params, args, kwargs)

    def run_node(self, n: fx.Node):
        out = super().run_node(n)
        first = out[0] if isinstance(out, (tuple, list)) and out else out
        if isinstance(first, torch.Tensor):
            n.meta["shape"], n.meta["dtype"], n.meta["numel"] = tuple(first.shape), first.dtype, first.numel()
        n.meta["flops"] = self._flops(n, out)
        return out

    def _flops(self, n: fx.Node, out) -> float:
        if n.op == "call_module":
            m = self.module.get_submodule(n.target)
            if isinstance(m, nn.Linear) and isinstance(out, torch.Tensor):
                return 2.0 * out.numel() * m.in_features
        if n.op in ("call_function", "call_method") and getattr(n.target, "__name__", n.target) in ("matmul", "bmm"):
            a = self.env[n.args[0]] if isinstance(n.args[0], fx.Node) else None
            if isinstance(a, torch.Tensor) and isinstance(out, torch.Tensor):
                return 2.0 * out.numel() * a.shape[-1]
        return 0.0

    def propagate(self, *args, **kwargs):
        return self.run(*tree_map(_to_meta, args), **tree_map(_to_meta, kwargs)) if kwargs else \
            self.run(*tree_map(_to_meta, args))
