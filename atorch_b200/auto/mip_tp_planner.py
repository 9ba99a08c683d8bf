"""Tensor-parallel layout of a traced model as a mixed-integer programme.

Every ``nn.Linear`` / ``nn.Embedding`` leaf ``n`` of the fx graph gets one binary variable per layout
``s ∈ {replicate, col, row}``; every dataflow edge between two such leaves (paths through layout-keeping ops
are contracted) gets variables ``y[e, s, t]`` that equal ``x[u, s] · x[v, t]`` through the usual flow
constraints ``Σ_t y = x[u, s]``, ``Σ_s y = x[v, t]``. The objective is the time of one forward+backward pass:

* compute of a leaf: ``3 · flops / peak``, divided by the tensor-parallel size when the leaf is split;
* communication on an edge: what the producer's output layout (col → last-dimension split, row → partial sum,
  replicate → complete) costs to become what the consumer needs (col / replicate → complete, row → split),
  priced by ``SimpleTopology``: all-gather for split→complete, all-reduce for partial→complete,
  reduce-scatter for partial→split; an edge that passes a normalisation or leaves the graph needs a complete
  tensor; the backward pass pays the conjugate collective, so each cost counts twice;

subject to an optional per-device parameter-memory budget. Solved exactly with ``scipy.optimize.milp``
(HiGHS). For a transformer block this reproduces the column→row pairing of attention and MLP whenever the
layers are large enough for the saved compute to beat the two all-reduces, and replication otherwise.
(Reference: atorch/auto/opt_lib/shard_planners/mip_tp_planner.py:34, base_tp_planner.py:11, utils.py:48-656,
which formulate the same choice with pyomo + GLPK.)"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.fx as fx
import torch.nn as nn

from ..utils.shape_prop import MetaShapeProp
from ..utils.spec_prop import ELEMENTWISE, LAYOUT_KEEPING, _name
from ..utils.tracer import trace_model
from .planner import SimpleTopology

LAYOUTS = ("replicate", "col", "row")


def _bytes(n: fx.Node) -> float:
    dt = n.meta.get("dtype", torch.float32)
    return float(n.meta.get("numel", 0)) * torch.empty((), dtype=dt).element_size()


class MIPTensorParallelPlanner:
    def __init__(self, tp_size: int, topology: Optional[SimpleTopology] = None, peak_flops: float = 1.4e15,
                 memory_budget_bytes: Optional[float] = None, ranks: Optional[List[int]] = None):
        self.tp = tp_size
        self.topo = topology or SimpleTopology(1, max(tp_size, 1), 770e9, 50e9)
        self.peak, self.budget = peak_flops, memory_budget_bytes
        self.ranks = ranks or list(range(tp_size))

    # ---------------------------------------------------------------- graph reduction
    def _leaves_and_edges(self, gm: fx.GraphModule):
        leaves = [n for n in gm.graph.nodes if n.op == "call_module"
                  and isinstance(gm.get_submodule(n.target), (nn.Linear, nn.Embedding))]
        leaf_set = set(leaves)
        edges: Dict[Tuple[fx.Node, fx.Node], bool] = {}      # (u, v) -> the path needs a complete tensor
        to_output: Dict[fx.Node, bool] = {}
        for u in leaves:
            stack = [(u, False)]
            seen = set()
            while stack:
                cur, needs_full = stack.pop()
                for user in cur.users:
                    key = (user, needs_full)
                    if key in seen:
                        continue
                    seen.add(key)
                    if user in leaf_set:
                        edges[(u, user)] = edges.get((u, user), False) or needs_full
                        continue
                    if user.op == "output":
                        to_output[u] = True
                        continue
                    nm = _name(user)
                    keeps = user.op != "call_module" and (nm in ELEMENTWISE or nm in LAYOUT_KEEPING)
                    stack.append((user, needs_full or not keeps))
        return leaves, edges, to_output

    # ---------------------------------------------------------------- costs
    def _ar(self, nbytes: float) -> float:
        return self.topo.all_reduce_time(nbytes, self.ranks)

    def _edge_cost(self, u: fx.Node, s: str, t: str, needs_full: bool) -> float:
        b = _bytes(u)
        ar = self._ar(b)
        ag = rs = ar / 2.0
        want_split = (t == "row") and not needs_full
        if s == "col":                      # last dimension split
            c = 0.0 if want_split else ag
            if needs_full and t == "row":
                c = ag                     # gathered for the op in between, sliced again for free
        elif s == "row":                    # partial sum
            c = rs if want_split else ar
        else:
            c = 0.0
        return 2.0 * c                      # forward + the conjugate collective of the backward pass

    def _node_cost(self, gm, n: fx.Node, s: str) -> Tuple[float, float]:
        m = gm.get_submodule(n.target)
        flops = float(n.meta.get("flops", 0.0))
        pbytes = float(sum(p.numel() * p.element_size() for p in m.parameters()))
        div = self.tp if s != "replicate" else 1
        return 3.0 * flops / self.peak / div, pbytes / div

    def _divisible(self, gm, n: fx.Node, s: str) -> bool:
        m = gm.get_submodule(n.target)
        if s == "replicate":
            return True
        if isinstance(m, nn.Linear):
            return (m.out_features if s == "col" else m.in_features) % self.tp == 0
        return (m.embedding_dim if s == "col" else m.num_embeddings) % self.tp == 0

    # ---------------------------------------------------------------- solve
    def plan_graph(self, gm: fx.GraphModule) -> Dict[str, str]:
        from scipy.optimize import Bounds, LinearConstraint, milp

        leaves, edges, to_output = self._leaves_and_edges(gm)
        if not leaves:
            return {}
        nx = 3 * len(leaves)
        idx = {n: 3 * i for i, n in enumerate(leaves)}
        elist = list(edges.items())
        ny = 9 * len(elist)
        c = np.zeros(nx + ny)
        ub = np.ones(nx + ny)
        mem_row = np.zeros(nx + ny)
        for n in leaves:
            for k, s in enumerate(LAYOUTS):
                t, mem = self._node_cost(gm, n, s)
                if s == "row" and to_output.get(n):          # a partial sum leaving the graph is reduced
                    t += 2.0 * self._ar(_bytes(n))
                if s == "col" and to_output.get(n):
                    t += self._ar(_bytes(n))                 # gathered: all-gather fwd + reduce-scatter bwd
                c[idx[n] + k] = t
                mem_row[idx[n] + k] = mem
                if not self._divisible(gm, n, s):
                    ub[idx[n] + k] = 0.0
        rows, lo, hi = [], [], []
        for n in leaves:                                       # one layout per leaf
            r = np.zeros(nx + ny)
            r[idx[n]: idx[n] + 3] = 1.0
            rows.append(r); lo.append(1.0); hi.append(1.0)
        for e, ((u, v), needs_full) in enumerate(elist):
            base = nx + 9 * e
            for si, s in enumerate(LAYOUTS):
                for ti, t in enumerate(LAYOUTS):
                    c[base + 3 * si + ti] = self._edge_cost(u, s, t, needs_full)
            for si in range(3):                                # Σ_t y[s, t] = x[u, s]
                r = np.zeros(nx + ny)
                r[base + 3 * si: base + 3 * si + 3] = 1.0
                r[idx[u] + si] = -1.0
                rows.append(r); lo.append(0.0); hi.append(0.0)
            for ti in range(3):                                # Σ_s y[s, t] = x[v, t]
                r = np.zeros(nx + ny)
                r[[base + ti, base + 3 + ti, base + 6 + ti]] = 1.0
                r[idx[v] + ti] = -1.0
                rows.append(r); lo.append(0.0); hi.append(0.0)
        if self.budget is not None:
            rows.append(mem_row); lo.append(0.0); hi.append(float(self.budget))
        scale = float(c.max()) or 1.0           # seconds of 1e-9 would sit below the solver's tolerances
        res = milp(c / scale, constraints=LinearConstraint(np.array(rows), np.array(lo), np.array(hi)),
                   integrality=np.ones(nx + ny), bounds=Bounds(np.zeros(nx + ny), ub))
        if not res.success:
            raise RuntimeError(f"no feasible tensor-parallel layout: {res.message}")
        self.objective = float(res.fun) * scale
        out = {}
        for n in leaves:
            k = int(np.argmax(res.x[idx[n]: idx[n] + 3]))
            out[n.target] = LAYOUTS[k]
        return out

    def plan(self, model: nn.Module, example_inputs: Tuple, concrete_args=None) -> Dict[str, str]:
        gm = trace_model(model, concrete_args)
        MetaShapeProp(gm).propagate(*example_inputs)
        self.graph_module = gm
        return self.plan_graph(gm)
