"""Tensor-parallel layers: ``ColumnParallelLinear``, ``RowParallelLinear``, ``VocabParallelEmbedding``.

Weights are created from an existing ``nn.Linear`` / ``nn.Embedding`` (``orig_module``), each rank
keeping its slice (``stride`` handles fused projections such as q|k|v: every one of the ``stride``
sub-matrices is sliced separately).

Two communication styles:
* all-reduce style (the reference's own layers): column = identity fwd / all-reduce bwd, row =
  all-reduce fwd;
* ``sequence_parallel=True`` (Megatron style, which the reference only reaches through Megatron):
  activations outside the TP block are sharded along the sequence dim; column = all-gather(seq)
  then GEMM, row = GEMM then reduce-scatter(seq).

  On 2..8 GPUs of one NVSwitch domain each of these is ONE GEMM launch fused with its collective
  (``ops/tp_fused.py``: arrival-flag gated all-gather -> GEMM, GEMM -> reduce-scatter in the epilogue over
  peer pointers); elsewhere ``torch.distributed`` collectives surround the GEMM.

The GEMMs run on ``ops.linear`` (tcgen05 kernel on the GPU).
(Reference: atorch/modules/distributed_modules/layers.py:90-760.)
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ... import ops
from ...distributed import distributed as D
from .mappings import (all_gather_from_group, copy_to_group, gather_from_group, reduce_from_group,
                       reduce_scatter_to_group, scatter_to_group)


def _group(pg):
    if isinstance(pg, str):
        return D.parallel_group(pg)
    return pg


def _ws(g):
    return dist.get_world_size(g) if (dist.is_available() and dist.is_initialized()) else 1


def _rk(g):
    return dist.get_rank(g) if (dist.is_available() and dist.is_initialized()) else 0


def _fusable(x: torch.Tensor, weight: torch.Tensor, group, rows_local: int, n: int, k: int) -> bool:
    """May the fused collective+GEMM kernels take this call? (bf16 on CUDA, one sequence per call, whole
    256-row tiles per shard, peer memory available, not switched off with ATB_FUSED_COMM=0)"""
    import os

    if not (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16) or \
            os.environ.get("ATB_FUSED_COMM", "1") == "0":
        return False
    if any(d != 1 for d in x.shape[:-2]):
        return False
    from ...ops import tp_fused

    return tp_fused.shapes_ok(rows_local, n, k) and tp_fused.available(group)


def _slice_rows(w: torch.Tensor, rank: int, world: int, stride: int = 1) -> torch.Tensor:
    """Rows owned by ``rank`` of a weight whose rows are ``stride`` stacked blocks."""
    if world == 1:
        return w.clone()
    blocks = w.chunk(stride, dim=0)
    return torch.cat([b.chunk(world, dim=0)[rank] for b in blocks], dim=0).contiguous()


class ColumnParallelLinear(nn.Module):
    """``Y = X A^T`` with the output features (rows of ``A``) split over the group."""

    def __init__(self, in_features: Optional[int] = None, out_features: Optional[int] = None, bias: bool = True,
                 orig_module: Optional[nn.Linear] = None, process_group="tensor", ranks=None,
                 gather_output: bool = False, stride: int = 1, sequence_parallel: bool = False,
                 defer_init: bool = False, dtype=None, device=None):
        super().__init__()
        self.group = _group(process_group)
        self.world, self.rank = _ws(self.group), _rk(self.group)
        if orig_module is not None:
            in_features, out_features = orig_module.in_features, orig_module.out_features
            bias = orig_module.bias is not None
            dtype = dtype or orig_module.weight.dtype
            device = device or orig_module.weight.device
        assert out_features % (self.world * stride) == 0, "out_features must divide by tp size * stride"
        self.in_features, self.out_features = in_features, out_features
        self.out_per_rank = out_features // self.world
        self.gather_output, self.stride, self.sequence_parallel = gather_output, stride, sequence_parallel
        dev = "meta" if defer_init else device
        self.weight = nn.Parameter(torch.empty(self.out_per_rank, in_features, dtype=dtype, device=dev))
        self.bias = nn.Parameter(torch.empty(self.out_per_rank, dtype=dtype, device=dev)) if bias else None
        if orig_module is not None and not defer_init and not orig_module.weight.is_meta:
            with torch.no_grad():
                self.weight.copy_(_slice_rows(orig_module.weight.detach(), self.rank, self.world, stride))
                if bias:
                    self.bias.copy_(_slice_rows(orig_module.bias.detach()[:, None], self.rank, self.world, stride)[:, 0])
        elif not defer_init:
            self.reset_parameters()

    def reset_parameters(self):
        nn.init.normal_(self.weight, std=0.02)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, x):
        if self.sequence_parallel and self.world > 1 and x.dim() >= 2 and \
                _fusable(x, self.weight, self.group, x.shape[-2], self.out_per_rank, self.in_features):
            from ...ops.tp_fused import allgather_linear

            y = allgather_linear(x, self.weight, self.group)      # all-gather(seq) fused into the GEMM
            if self.bias is not None:
                y = y + self.bias
            if self.gather_output:
                y = gather_from_group(y, self.group, dim=-1)
            return y
        if self.sequence_parallel:
            x = all_gather_from_group(x, self.group, dim=x.dim() - 2)
        else:
            x = copy_to_group(x, self.group)
        y = ops.linear(x, self.weight, self.bias)
        if self.gather_output:
            y = gather_from_group(y, self.group, dim=-1)
        return y


class RowParallelLinear(nn.Module):
    """``Y = X A^T`` with the input features (columns of ``A``) split over the group."""

    def __init__(self, in_features: Optional[int] = None, out_features: Optional[int] = None, bias: bool = True,
                 orig_module: Optional[nn.Linear] = None, process_group="tensor", ranks=None,
                 input_is_parallel: bool = True, sequence_parallel: bool = False, defer_init: bool = False,
                 dtype=None, device=None):
        super().__init__()
        self.group = _group(process_group)
        self.world, self.rank = _ws(self.group), _rk(self.group)
        if orig_module is not None:
            in_features, out_features = orig_module.in_features, orig_module.out_features
            bias = orig_module.bias is not None
            dtype = dtype or orig_module.weight.dtype
            device = device or orig_module.weight.device
        assert in_features % self.world == 0
        self.in_features, self.out_features = in_features, out_features
        self.in_per_rank = in_features // self.world
        self.input_is_parallel, self.sequence_parallel = input_is_parallel, sequence_parallel
        dev = "meta" if defer_init else device
        self.weight = nn.Parameter(torch.empty(out_features, self.in_per_rank, dtype=dtype, device=dev))
        self.bias = nn.Parameter(torch.empty(out_features, dtype=dtype, device=dev)) if bias else None
        if orig_module is not None and not defer_init and not orig_module.weight.is_meta:
            with torch.no_grad():
                self.weight.copy_(orig_module.weight.detach().chunk(self.world, dim=1)[self.rank])
                if bias:
                    self.bias.copy_(orig_module.bias.detach())
        elif not defer_init:
            self.reset_parameters()

    def reset_parameters(self):
        nn.init.normal_(self.weight, std=0.02)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, x):
        if not self.input_is_parallel:
            x = scatter_to_group(x, self.group, dim=-1)
        if self.sequence_parallel and self.world > 1 and x.dim() >= 2 and x.shape[-2] % self.world == 0 and \
                _fusable(x, self.weight, self.group, x.shape[-2] // self.world, self.out_features, self.in_per_rank):
            from ...ops.tp_fused import linear_reduce_scatter

            y = linear_reduce_scatter(x, self.weight, self.group)  # reduce-scatter(seq) in the GEMM epilogue
            return y if self.bias is None else y + self.bias
        y = ops.linear(x, self.weight)
        if self.sequence_parallel:
            y = reduce_scatter_to_group(y, self.group, dim=y.dim() - 2)
        else:
            y = reduce_from_group(y, self.group)
        if self.bias is not None:
            y = y + self.bias
        return y


class VocabParallelEmbedding(nn.Module):
    """Embedding table split along the vocabulary; out-of-range ids contribute zeros, then all-reduce."""

    def __init__(self, num_embeddings: Optional[int] = None, embedding_dim: Optional[int] = None,
                 orig_module: Optional[nn.Embedding] = None, process_group="tensor", ranks=None,
                 defer_init: bool = False, dtype=None, device=None, padding_idx=None):
        super().__init__()
        self.group = _group(process_group)
        self.world, self.rank = _ws(self.group), _rk(self.group)
        if orig_module is not None:
            num_embeddings, embedding_dim = orig_module.num_embeddings, orig_module.embedding_dim
            dtype = dtype or orig_module.weight.dtype
            device = device or orig_module.weight.device
            padding_idx = orig_module.padding_idx
        assert num_embeddings % self.world == 0
        self.num_embeddings, self.embedding_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.per_rank = num_embeddings // self.world
        self.vocab_start, self.vocab_end = self.rank * self.per_rank, (self.rank + 1) * self.per_rank
        dev = "meta" if defer_init else device
        self.weight = nn.Parameter(torch.empty(self.per_rank, embedding_dim, dtype=dtype, device=dev))
        if orig_module is not None and not defer_init and not orig_module.weight.is_meta:
            with torch.no_grad():
                self.weight.copy_(orig_module.weight.detach()[self.vocab_start: self.vocab_end])
        elif not defer_init:
            nn.init.normal_(self.weight, std=0.02)

    def forward(self, ids):
        if self.world == 1:
            return nn.functional.embedding(ids, self.weight, self.padding_idx)
        mask = (ids < self.vocab_start) | (ids >= self.vocab_end)
        local = (ids - self.vocab_start).masked_fill(mask, 0)
        out = nn.functional.embedding(local, self.weight)
        out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        return reduce_from_group(out, self.group)
