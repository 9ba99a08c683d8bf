"""Topology-aware node rank ordering: given each node's switch / rack labels, order nodes so that
consecutive ranks share a switch (ring and tree collectives then cross as few uplinks as possible).
(Reference: atorch/utils/rank_reorder.py, used with k8s top-of-rack labels.)"""
from __future__ import annotations

from typing import Dict, List, Sequence


def reorder_nodes_by_topology(node_labels: Sequence[Dict[str, str]], keys: Sequence[str] = ("pod", "rack", "switch")
                              ) -> List[int]:
    """Returns the new order (a permutation of node indices), stable inside identical label tuples."""
    def label(i):
        return tuple(node_labels[i].get(k, "") for k in keys)
    return sorted(range(len(node_labels)), key=lambda i: (label(i), i))


def new_node_rank(node_index: int, node_labels: Sequence[Dict[str, str]], keys=("pod", "rack", "switch")) -> int:
    return reorder_nodes_by_topology(node_labels, keys).index(node_index)
