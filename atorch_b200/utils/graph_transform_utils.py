"""Helpers for fx-graph rewrites: a topological sort of a node subset and structure-preserving maps over nested
arguments. (Reference: atorch/utils/graph_transform_utils.py:58-142.)"""
from collections import deque


def topo_sort(nodes):
    """Nodes (``torch.fx.Node``s, or anything with ``all_input_nodes`` and ``users``) in dependency order; edges to
    nodes outside the subset are ignored."""
    members = set(nodes)
    indegree = {n: sum(1 for i in n.all_input_nodes if i in members) for n in nodes}
    ready = deque(n for n in nodes if indegree[n] == 0)
    order = []
    while ready:
        n = ready.popleft()
        order.append(n)
        for u in n.users:
            if u in indegree:
                indegree[u] -= 1
                if indegree[u] == 0:
                    ready.append(u)
    assert len(order) == len(nodes), "topological sorted nodes doesn't have same length as input nodes"
    return order


def map_aggregate(input_, fn):
    """``fn`` applied to every leaf of nested tuples (named tuples keep their type), lists, dicts and slices."""
    if isinstance(input_, tuple):
        mapped = tuple(map_aggregate(e, fn) for e in input_)
        return type(input_)(*mapped) if hasattr(input_, "_fields") else mapped
    if isinstance(input_, list):
        return [map_aggregate(e, fn) for e in input_]
    if isinstance(input_, dict):
        return {k: map_aggregate(v, fn) for k, v in input_.items()}
    if isinstance(input_, slice):
        return slice(map_aggregate(input_.start, fn), map_aggregate(input_.stop, fn), map_aggregate(input_.step, fn))
    return fn(input_)


def combine_map_aggregate(input_0, input_1, fn):
    """Walks two equally shaped structures together and calls ``fn(a, b)`` on the leaf pairs for its side effect on
    ``a`` (e.g. ``a.copy_(b)``); returns ``input_0``. Lists and dicts of ``input_0`` are walked in place; tuples and
    slices are rebuilt from the (unchanged or mutated) leaves."""
    if isinstance(input_0, tuple) and isinstance(input_1, tuple):
        return tuple(combine_map_aggregate(a, b, fn) for a, b in zip(input_0, input_1))
    if isinstance(input_0, list) and isinstance(input_1, list):
        for i in range(len(input_0)):
            input_0[i] = combine_map_aggregate(input_0[i], input_1[i], fn)
        return input_0
    if isinstance(input_0, dict) and isinstance(input_1, dict):
        for k in input_0:
            input_0[k] = combine_map_aggregate(input_0[k], input_1[k], fn)
        return input_0
    if isinstance(input_0, slice) and isinstance(input_1, slice):
        return slice(combine_map_aggregate(input_0.start, input_1.start, fn),
                     combine_map_aggregate(input_0.stop, input_1.stop, fn),
                     combine_map_aggregate(input_0.step, input_1.step, fn))
    fn(input_0, input_1)
    return input_0
