"""``all_reduce_sparse``: sum a sparse COO tensor over a group by all-gathering padded (indices, values)
and coalescing (reference: atorch/utils/sparse.py:6-61)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def all_reduce_sparse(t: torch.Tensor, group=None) -> torch.Tensor:
    t = t.coalesce()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return t
    idx, val = t.indices(), t.values()
    n = torch.tensor([idx.shape[1]], device=idx.device)
    sizes = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(sizes, n, group=group)
    m = int(max(s.item() for s in sizes))
    pad_i = torch.zeros(idx.shape[0], m, dtype=idx.dtype, device=idx.device)
    pad_v = torch.zeros((m,) + tuple(val.shape[1:]), dtype=val.dtype, device=val.device)
    pad_i[:, : idx.shape[1]] = idx
    pad_v[: val.shape[0]] = val
    all_i = [torch.empty_like(pad_i) for _ in range(world)]
    all_v = [torch.empty_like(pad_v) for _ in range(world)]
    dist.all_gather(all_i, pad_i, group=group)
    dist.all_gather(all_v, pad_v, group=group)
    ii = torch.cat([a[:, : int(s.item())] for a, s in zip(all_i, sizes)], dim=1)
    vv = torch.cat([a[: int(s.item())] for a, s in zip(all_v, sizes)], dim=0)
    return torch.sparse_coo_tensor(ii, vv, t.shape).coalesce()
