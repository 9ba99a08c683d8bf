"""GLM mask constructions under the names the NPU attention layer of the original package exports. They return the
visibility matrix as a float tensor ``[B, 1, S, S]`` with 1 = may attend (the flash kernels of this package take the
same information as per-row key intervals, ``ops.flash.row_intervals``).
(Reference: atorch/npu/layers.py:9-56.)
"""
from __future__ import annotations

import torch

from ..modules.transformer.rmsnorm import AtorchRmsNorm
from ..ops.attention import build_dense_mask


def create_additive_mask_by_breakpoint_mask(batch_size: int, seq_length: int, glm_mask: torch.Tensor) -> torch.Tensor:
    """Causal, plus every key before the break point visible to all queries. ``glm_mask``: one break point for the
    whole batch (a one-element tensor; the result then has batch size 1 and broadcasts) or one per sample."""
    if glm_mask.numel() == 1:
        batch_size, glm_mask = 1, glm_mask.reshape(1)
    vis = build_dense_mask(batch_size, seq_length, seq_length, glm_mask.device, True, glm_mask, None, None, None)
    return vis.to(torch.float32)


def create_additive_pack_mask_by_startpoint_endpoint_mask(batch_size: int, seq_length: int,
                                                          pack_glm_mask: torch.Tensor) -> torch.Tensor:
    """Causal, plus for every (start, end) pair of a sample: queries from ``start`` on see all keys before ``end``.
    ``pack_glm_mask``: ``[B, 2, n]`` (row 0 starts, row 1 ends)."""
    assert pack_glm_mask.dim() == 3
    vis = build_dense_mask(batch_size, seq_length, seq_length, pack_glm_mask.device, True, None, pack_glm_mask, None,
                           None)
    return vis.to(torch.float32)


def delete_minus_one_in_pack_glm_mask(pack_glm_mask: torch.Tensor, invalid_point: int = -1) -> torch.Tensor:
    """One sample's ``[2, n]`` pairs cut at the first column that holds the padding value."""
    bad = (pack_glm_mask == invalid_point).any(dim=0)
    if not bad.any():
        return pack_glm_mask
    return pack_glm_mask[:, : int(bad.to(torch.int32).argmax())]


AtorchNpuRMSNorm = AtorchRmsNorm
