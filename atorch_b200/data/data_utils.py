"""Batch helpers for the strategy search (reference: atorch/data/data_utils.py)."""
from __future__ import annotations

import torch


def get_sample_batch(dataset, dataloader_args=None, num: int = 1):
    """A collated batch of the first ``num`` samples of ``dataset``."""
    args = dict(dataloader_args or {})
    collate = args.get("collate_fn") or torch.utils.data.default_collate
    return collate([dataset[i] for i in range(min(num, len(dataset)))])


def expand_batch_dim(data, batch_size: int = 1):
    """Add a leading batch dim of ``batch_size`` to every tensor of a (nested) sample."""
    if isinstance(data, torch.Tensor):
        return data.unsqueeze(0).expand(batch_size, *data.shape).contiguous()
    if isinstance(data, dict):
        return {k: expand_batch_dim(v, batch_size) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(expand_batch_dim(v, batch_size) for v in data)
    if isinstance(data, (int, float)):
        return torch.tensor([data] * batch_size)
    return data
