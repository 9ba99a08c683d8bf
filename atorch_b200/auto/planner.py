"""Choosing (tensor, pipeline, data) sizes and pipeline stage boundaries for a model on a machine.

``DimPlanner.generate_sharding_plan`` enumerates tensor sizes (powers of two up to the GPUs of a
node) and pipeline sizes dividing the rest, in increasing model-parallel product, estimates per-stage
memory (weights + optimizer state / dp-shard + in-flight activations) and step time (compute at the
measured GEMM throughput, tensor-parallel all-reduces and pipeline bubbles over NVLink), and keeps
the first feasible candidate. ``tera_pipe_partition`` is the dynamic programme that splits a sequence
of layer costs into stages minimising ``(stages - 1) * max_stage + sum`` under a memory cap.
(Reference: atorch/auto/opt_lib/shard_planners/dim_planner.py:17-238, base_stage_planner.py:125,
topology.py:4-82, mixed_parallel_optimization.py:32-307.)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch.nn as nn

from .device_context import get_device_context


class SimpleTopology:
    """Full mesh inside a node at ``intra_bw``, full mesh between nodes at ``inter_bw`` (bytes/s)."""

    def __init__(self, num_nodes: int, gpus_per_node: int, intra_bw: float, inter_bw: float):
        self.num_nodes, self.gpus_per_node, self.intra_bw, self.inter_bw = num_nodes, gpus_per_node, intra_bw, inter_bw

    def effective_bandwidth(self, ranks: Sequence[int]) -> float:
        nodes = {r // self.gpus_per_node for r in ranks}
        return self.intra_bw if len(nodes) <= 1 else self.inter_bw

    def all_reduce_time(self, nbytes: float, ranks: Sequence[int]) -> float:
        n = len(ranks)
        return 0.0 if n <= 1 else 2.0 * nbytes * (n - 1) / n / self.effective_bandwidth(ranks)


def tera_pipe_partition(costs: Sequence[float], mems: Sequence[float], num_stages: int,
                        mem_cap: float = math.inf) -> Optional[List[int]]:
    """Split ``len(costs)`` consecutive layers into ``num_stages`` stages; returns the layer count of
    every stage minimising ``(num_stages - 1) * max_stage_cost + total`` subject to the memory cap."""
    n = len(costs)
    pre_c, pre_m = [0.0], [0.0]
    for c, m in zip(costs, mems):
        pre_c.append(pre_c[-1] + c)
        pre_m.append(pre_m[-1] + m)
    best = None
    for tmax in sorted({pre_c[j] - pre_c[i] for i in range(n) for j in range(i + 1, n + 1)}):
        # greedy feasibility for this cap on the largest stage: fewest stages with cost <= tmax and mem <= cap
        sizes, i = [], 0
        ok = True
        while i < n:
            j = i
            while j < n and pre_c[j + 1] - pre_c[i] <= tmax + 1e-12 and pre_m[j + 1] - pre_m[i] <= mem_cap:
                j += 1
            if j == i:
                ok = False
                break
            sizes.append(j - i)
            i = j
        if not ok or len(sizes) > num_stages:
            continue
        while len(sizes) < num_stages:                      # split the largest stage until the count fits
            k = max(range(len(sizes)), key=lambda t: sizes[t])
            if sizes[k] < 2:
                break
            sizes[k: k + 1] = [sizes[k] - sizes[k] // 2, sizes[k] // 2]
        if len(sizes) == num_stages:
            stage_costs, pos = [], 0
            for s in sizes:
                stage_costs.append(pre_c[pos + s] - pre_c[pos])
                pos += s
            obj = (num_stages - 1) * max(stage_costs) + sum(stage_costs)
            if best is None or obj < best[0]:
                best = (obj, sizes)
            break
    return best[1] if best else None


def layer_costs(model: nn.Module, block_cls=None, tokens_per_batch: int = 4096) -> Tuple[List[float], List[float]]:
    """Per-block (forward FLOPs, parameter bytes) of the repeated block class (or of top-level children)."""
    blocks = [m for m in model.modules() if block_cls is not None and isinstance(m, block_cls)] or \
        list(model.children())
    flops, mem = [], []
    for b in blocks:
        p = sum(x.numel() for x in b.parameters())
        flops.append(2.0 * p * tokens_per_batch)
        mem.append(p * 2.0)
    return flops, mem


class DimPlanner:
    def __init__(self, num_nodes: Optional[int] = None, num_devices_per_node: Optional[int] = None,
                 memory_bound: Optional[float] = None, flops: Optional[float] = None):
        dc = get_device_context()
        self.num_nodes = num_nodes or dc.node_num
        self.gpus = num_devices_per_node or max(dc.nproc_per_node, 1)
        self.memory_bound = memory_bound or (dc.gpu_memory * 0.9 if dc.gpu_memory else 160e9)
        self.flops = flops or dc.bf16_flops
        self.topology = SimpleTopology(self.num_nodes, self.gpus, dc.intra_node_bandwidth, dc.inter_node_bandwidth)

    def candidates(self) -> List[Tuple[int, int, int]]:
        world = self.num_nodes * self.gpus
        out = []
        t = 1
        while t <= self.gpus:
            rest = world // t
            for p in range(1, rest + 1):
                if rest % p == 0:
                    out.append((t, p, rest // p))
            t *= 2
        return sorted(out, key=lambda c: (c[0] * c[1], c[0]))

    def estimate(self, flops: List[float], mems: List[float], tensor: int, pipe: int, data: int,
                 micro_batches: int = 8, activation_bytes_per_layer: float = 64e6):
        sizes = tera_pipe_partition(flops, mems, pipe, math.inf) or [len(flops) // pipe] * pipe
        pos, stage_mem, stage_time = 0, [], []
        for s in sizes:
            w = sum(mems[pos: pos + s]) / tensor
            state = w * 6.0 / max(data, 1) + w            # fp32 master + 2 moments sharded over data, bf16 copy resident
            act = activation_bytes_per_layer * s * min(pipe, micro_batches) / tensor
            stage_mem.append(state + act)
            comp = 3.0 * sum(flops[pos: pos + s]) / tensor / self.flops
            comm = 4 * s * self.topology.all_reduce_time(activation_bytes_per_layer / 4, list(range(tensor)))
            stage_time.append(comp + comm)
            pos += s
        bubble = (pipe - 1) * max(stage_time)
        return max(stage_mem), micro_batches * max(stage_time) + bubble, sizes

    def generate_sharding_plan(self, model: nn.Module, block_cls=None, micro_batches: int = 8,
                               tokens_per_batch: int = 4096, activation_bytes_per_layer: float = 64e6) -> Dict:
        flops, mems = layer_costs(model, block_cls, tokens_per_batch)
        best = None
        for t, p, d in self.candidates():
            if p > len(flops):
                continue
            mem, time_, sizes = self.estimate(flops, mems, t, p, d, micro_batches, activation_bytes_per_layer)
            if mem <= self.memory_bound:
                cand = {"tensor": t, "pipe": p, "data": d, "stage_layers": sizes, "est_memory": mem,
                        "est_step_time": time_ / max(d, 1)}
                if best is None or cand["est_step_time"] < best["est_step_time"] * 0.95:
                    best = cand
                if best is not None and t * p > best["tensor"] * best["pipe"] * 4:
                    break
        return best or {"tensor": 1, "pipe": 1, "data": self.num_nodes * self.gpus, "stage_layers": [len(flops)]}


def plan_mixed_parallel(model_context, config: Optional[dict] = None) -> dict:
    """Config for the ``mixed_parallel`` optimisation: sizes from ``parallel_mode`` when given, else planned."""
    from .analyser import analyse_model

    config = dict(config or {})
    model = model_context.model
    block = (analyse_model(model).get("opt_config_submodule_names") or (None,))[0]
    pm = model_context.parallel_mode_config
    if pm is not None:
        sizes = dict(pm[0])
        plan = {"tensor": sizes.get("tensor", 1), "pipe": sizes.get("pipe", sizes.get("pipeline", 1)),
                "data": sizes.get("data", 1)}
    else:
        plan = DimPlanner().generate_sharding_plan(model, block)
    out = {"plan": plan}
    if plan["tensor"] > 1:
        out["tensor_parallel"] = config.get("tensor_parallel", {})
    if plan["pipe"] > 1:
        out["pipeline_parallel"] = dict(config.get("pipeline_parallel", {}), stage_layers=plan.get("stage_layers"))
    return out
