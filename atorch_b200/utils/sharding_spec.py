"""Sharding specifications of tensors over a device mesh and the cost of converting between them.

``MeshShardingSpec(dims, partial)``: ``dims[i]`` is the mesh axis that tensor dimension ``i`` is split over, or
``-1`` for a replicated dimension; ``partial`` names mesh axes over which the tensor is a partial sum (an
all-reduce away from its value). ``reshard_plan(src, dst)`` lists the collectives that turn one into the
other — slicing is free, un-splitting is an all-gather, partial→replicated an all-reduce, partial→split a
reduce-scatter, moving a split from one dimension to another an all-to-all — and ``reshard_time`` prices the
list with a bandwidth model. (Reference: atorch/utils/sharding_spec.py, spec_prop.py.)"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple


@dataclass(frozen=True)
class MeshShardingSpec:
    dims: Tuple[int, ...]
    partial: Tuple[int, ...] = field(default_factory=tuple)

    @staticmethod
    def replicated(ndim: int) -> "MeshShardingSpec":
        return MeshShardingSpec((-1,) * ndim)

    @staticmethod
    def split(ndim: int, tensor_dim: int, mesh_axis: int = 0) -> "MeshShardingSpec":
        d = [-1] * ndim
        d[tensor_dim % ndim] = mesh_axis
        return MeshShardingSpec(tuple(d))

    def is_replicated(self) -> bool:
        return all(d < 0 for d in self.dims) and not self.partial

    def split_dim(self, mesh_axis: int = 0) -> int:
        for i, d in enumerate(self.dims):
            if d == mesh_axis:
                return i
        return -1

    def shard_shape(self, shape: Sequence[int], mesh_shape: Sequence[int]) -> Tuple[int, ...]:
        out = []
        for s, d in zip(shape, self.dims):
            if d >= 0:
                assert s % mesh_shape[d] == 0, f"dimension of size {s} is not divisible by mesh axis {d}"
                s //= mesh_shape[d]
            out.append(s)
        return tuple(out)


def reshard_plan(src: MeshShardingSpec, dst: MeshShardingSpec, mesh_axis: int = 0) -> List[str]:
    """Collectives along one mesh axis, in order."""
    ops: List[str] = []
    s, d = src.split_dim(mesh_axis), dst.split_dim(mesh_axis)
    partial = mesh_axis in src.partial
    if mesh_axis in dst.partial and not partial:
        raise ValueError("a complete tensor cannot become a partial sum")
    if partial and mesh_axis not in dst.partial:
        if d >= 0 and s < 0:
            return ["reduce_scatter"]
        ops.append("all_reduce")
    if s == d:
        return ops
    if s >= 0 and d >= 0:
        ops.append("all_to_all")
    elif s >= 0:
        ops.append("all_gather")
    # s < 0 <= d: every rank keeps its slice, no communication
    return ops


def collective_time(op: str, full_bytes: float, n: int, bandwidth: float, latency: float = 5e-6) -> float:
    """Ring / pairwise cost of a collective on ``n`` ranks for a tensor of ``full_bytes`` (unsharded size)."""
    if n <= 1:
        return 0.0
    f = (n - 1) / n
    vol = {"all_reduce": 2 * f * full_bytes, "all_gather": f * full_bytes, "reduce_scatter": f * full_bytes,
           "all_to_all": f * full_bytes / n}[op]
    return latency + vol / bandwidth


def reshard_time(src: MeshShardingSpec, dst: MeshShardingSpec, full_bytes: float, n: int, bandwidth: float,
                 mesh_axis: int = 0) -> float:
    return sum(collective_time(op, full_bytes, n, bandwidth) for op in reshard_plan(src, dst, mesh_axis))
