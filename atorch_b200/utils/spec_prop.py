"""``SpecProp``: propagate sharding specs through a traced graph.

Given the weight layout of every ``nn.Linear`` / ``nn.Embedding`` leaf (``"col"``: output features split,
``"row"``: input features split, ``"replicate"``), walk the graph in order and assign each node the
``MeshShardingSpec`` of its output, inserting the cheapest conversion where a consumer needs another layout;
the conversions are recorded as ``(node, input, [collectives])`` so a compiler can materialise them and a
planner can price them. Rules: a column-parallel linear wants a replicated input and yields a last-dimension
split; a row-parallel linear wants a last-dimension split and yields a partial sum; normalisations and
softmax over the last dimension, and anything unknown, want complete replicated inputs; element-wise ops keep
the layout of their (agreeing) inputs, otherwise replicate. (Reference: atorch/utils/spec_prop.py.)"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch.fx as fx
import torch.nn as nn

from .sharding_spec import MeshShardingSpec, reshard_plan

ELEMENTWISE = {"add", "mul", "sub", "truediv", "gelu", "silu", "relu", "tanh", "dropout", "sigmoid", "neg", "to",
               "float", "bfloat16", "half", "contiguous", "getitem", "type_as", "clone"}
LAYOUT_KEEPING = {"view", "reshape", "transpose", "permute", "matmul", "bmm", "scaled_dot_product_attention",
                  "unflatten", "flatten", "chunk", "split"}


def _name(n: fx.Node) -> str:
    return n.target if isinstance(n.target, str) else getattr(n.target, "__name__", str(n.target))


class SpecProp:
    def __init__(self, gm: fx.GraphModule, layouts: Dict[str, str], mesh_axis: int = 0):
        self.gm, self.layouts, self.axis = gm, layouts, mesh_axis
        self.specs: Dict[fx.Node, MeshShardingSpec] = {}
        self.conversions: List[Tuple[fx.Node, fx.Node, List[str]]] = []

    def _ndim(self, n: fx.Node) -> int:
        return len(n.meta.get("shape", (0, 0, 0)))

    def _want(self, consumer: fx.Node, inp: fx.Node, spec: MeshShardingSpec) -> None:
        have = self.specs.get(inp)
        if have is None or have == spec:
            return
        plan = reshard_plan(have, spec, self.axis)
        if plan:
            self.conversions.append((consumer, inp, plan))

    def propagate(self) -> Dict[fx.Node, MeshShardingSpec]:
        for n in self.gm.graph.nodes:
            ins = [a for a in n.all_input_nodes]
            nd = self._ndim(n)
            rep = MeshShardingSpec.replicated(nd)
            if n.op in ("placeholder", "get_attr"):
                self.specs[n] = rep
                continue
            if n.op == "output":
                for a in ins:
                    self._want(n, a, MeshShardingSpec.replicated(self._ndim(a)))
                continue
            if n.op == "call_module":
                m = self.gm.get_submodule(n.target)
                lay = self.layouts.get(n.target, "replicate")
                if isinstance(m, (nn.Linear, nn.Embedding)) and lay != "replicate":
                    a = ins[0]
                    if lay == "col":
                        self._want(n, a, MeshShardingSpec.replicated(self._ndim(a)))
                        self.specs[n] = MeshShardingSpec.split(nd, -1, self.axis)
                    else:
                        if isinstance(m, nn.Linear):
                            self._want(n, a, MeshShardingSpec.split(self._ndim(a), -1, self.axis))
                        self.specs[n] = MeshShardingSpec((-1,) * nd, (self.axis,))
                    continue
                for a in ins:
                    self._want(n, a, MeshShardingSpec.replicated(self._ndim(a)))
                self.specs[n] = rep
                continue
            name = _name(n)
            in_specs = [self.specs[a] for a in ins if a in self.specs]
            split_in = [s for s in in_specs if s.split_dim(self.axis) >= 0]
            if name in ELEMENTWISE or name in LAYOUT_KEEPING:
                partial = [s for s in in_specs if self.axis in s.partial]
                if partial and name in ("add", "sub", "getitem", "to", "contiguous", "type_as", "clone") and \
                        len(partial) == len(in_specs):
                    self.specs[n] = MeshShardingSpec((-1,) * nd, (self.axis,))     # sums of partial sums stay partial
                    continue
                for a in ins:
                    if a in self.specs and self.axis in self.specs[a].partial:
                        self._want(n, a, MeshShardingSpec.replicated(self._ndim(a)))
                        self.specs[a] = MeshShardingSpec.replicated(self._ndim(a))
                if split_in and all(s.split_dim(self.axis) >= 0 or True for s in in_specs):
                    # the split travels with the data: last dimension for element-wise ops, the head
                    # dimension through the reshapes of attention (kept as "some dimension is split")
                    self.specs[n] = MeshShardingSpec.split(nd, -1, self.axis) if nd else rep
                else:
                    self.specs[n] = rep
                continue
            for a in ins:
                self._want(n, a, MeshShardingSpec.replicated(self._ndim(a)))
            self.specs[n] = rep
        return self.specs
