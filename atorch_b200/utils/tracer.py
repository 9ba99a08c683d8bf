"""fx tracing with meta tensors.

``MetaTracer`` is a ``torch.fx.Tracer`` that (a) treats chosen module classes (default: ``nn.Linear``,
``nn.Embedding``, norms, ``nn.Dropout``) as leaves so that a planner sees one node per layer, (b) records the
qualified module name of every ``call_module`` node and of the module that *owns* every other node
(``node.meta["module_path"]``), and (c) can attach concrete non-tensor arguments. ``trace_model`` returns a
``GraphModule``; ``MetaShapeProp`` (``utils/shape_prop.py``) then fills shapes without allocating memory.
Models with data-dependent Python control flow are not traceable; give ``concrete_args`` for flags.
(Reference: atorch/utils/tracer.py:173, which wraps the Hugging Face tracer.)"""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple, Type

import torch
import torch.fx as fx
import torch.nn as nn

DEFAULT_LEAVES: Tuple[Type[nn.Module], ...] = (nn.Linear, nn.Embedding, nn.LayerNorm, nn.Dropout, nn.Conv1d,
                                               nn.Conv2d)


class MetaTracer(fx.Tracer):
    def __init__(self, leaf_cls: Tuple[Type[nn.Module], ...] = DEFAULT_LEAVES, leaf_names: Tuple[str, ...] = ()):
        super().__init__()
        self.leaf_cls, self.leaf_names = tuple(leaf_cls), set(leaf_names)
        self._scope: list = []

    def is_leaf_module(self, m: nn.Module, module_qualified_name: str) -> bool:
        if isinstance(m, self.leaf_cls) or module_qualified_name in self.leaf_names:
            return True
        name = type(m).__name__.lower()
        if "norm" in name and not list(m.children()):
            return True
        return super().is_leaf_module(m, module_qualified_name)

    def call_module(self, m, forward, args, kwargs):
        self._scope.append(self.path_of_module(m))
        try:
            return super().call_module(m, forward, args, kwargs)
        finally:
            self._scope.pop()

    def create_node(self, kind, target, args, kwargs, name=None, type_expr=None):
        node = super().create_node(kind, target, args, kwargs, name, type_expr)
        node.meta["module_path"] = target if kind == "call_module" else (self._scope[-1] if self._scope else "")
        return node


def trace_model(model: nn.Module, concrete_args: Optional[Dict[str, Any]] = None,
                leaf_cls: Tuple[Type[nn.Module], ...] = DEFAULT_LEAVES, leaf_names: Tuple[str, ...] = ()) -> fx.GraphModule:
    tracer = MetaTracer(leaf_cls, leaf_names)
    graph = tracer.trace(model, concrete_args=concrete_args)
    return fx.GraphModule(tracer.root, graph, type(model).__name__)


def meta_like(t: torch.Tensor) -> torch.Tensor:
    return torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device="meta")
