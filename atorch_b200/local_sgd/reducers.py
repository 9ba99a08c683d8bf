"""Pseudo-gradient reducers for local SGD: weighted linear averaging and generalised task
arithmetic (sparsify -> weight -> sign-consensus mask -> normalise -> all-reduce).

``reduce_tensor`` works in place on one flat tensor (or a list, which is flattened, reduced and
scattered back). Per-replica weights may be turned into softmax weights over the group
(``weight_softmax_temperature``), exchanged with one all-gather of a scalar.
(Reference: atorch/local_sgd/utils/reduce_methods/{base.py:9-60, linear.py:9-34,
generalized_task_arithmetic.py:11-93, sparsify.py:12-56}.)
"""
from __future__ import annotations

from enum import Enum
from typing import Iterable, Optional, Union

import torch
import torch.distributed as dist


class SparsificationMethod(str, Enum):
    magnitude = "magnitude"
    random = "random"
    rescaled_random = "rescaled_random"


def magnitude(tensor: torch.Tensor, density: float) -> torch.Tensor:
    """Keeps the ``density`` fraction of entries with the largest magnitude, zeroes the rest."""
    return sparsify(tensor, density, "magnitude")


def bernoulli(tensor: torch.Tensor, density: float, rescale: bool = True) -> torch.Tensor:
    """Keeps every entry with probability ``density`` (and divides the survivors by it when ``rescale``)."""
    return sparsify(tensor, density, "rescaled_random" if rescale else "random")


def sparsify(t: torch.Tensor, density: float, method: str) -> torch.Tensor:
    if density >= 1 or method is None:
        return t
    method = getattr(method, "value", method)
    flat = t.view(-1)
    if method == "magnitude":
        k = int(density * flat.numel())
        assert k > 0, "density too small: nothing would be kept"
        w = flat.abs().float()
        thresh_idx = torch.topk(w, k, largest=True).indices
        mask = torch.zeros_like(flat)
        mask[thresh_idx] = 1
        return (flat * mask).view_as(t)
    if method in ("random", "rescaled_random"):
        work = flat.float() if (flat.device.type == "cpu" and flat.dtype == torch.float16) else flat
        mask = torch.bernoulli(torch.full_like(work, density))
        res = work * mask
        if method == "rescaled_random":
            res = res / density
        return res.to(t.dtype).view_as(t)
    raise NotImplementedError(method)


class TensorReducer:
    def __init__(self, process_group=None, weight_softmax_temperature: Optional[float] = None):
        self.process_group = process_group
        self.weight_softmax_temperature = weight_softmax_temperature

    def _refine_weight(self, device, dtype, weight=1.0, step_weight=1.0, step_weight_ratio=0.0, **_):
        if self.weight_softmax_temperature is not None:
            w = torch.as_tensor(weight, dtype=torch.float32, device=device).reshape(-1)[:1].clone()
            w = w / self.weight_softmax_temperature
            world = dist.get_world_size(self.process_group)
            allw = torch.empty(world, dtype=torch.float32, device=device)
            dist.all_gather_into_tensor(allw, w, group=self.process_group)
            w = torch.softmax(allw, dim=0)[dist.get_rank(self.process_group)]
        else:
            w = torch.as_tensor(weight, dtype=torch.float32, device=device)
        w = w * (1 - step_weight_ratio) + step_weight * step_weight_ratio
        return w.to(dtype)

    def _reduce_tensor(self, tensor: torch.Tensor, **kwargs) -> None:
        raise NotImplementedError

    @torch.no_grad()
    def reduce_tensor(self, tensors: Union[Iterable[torch.Tensor], torch.Tensor], **kwargs) -> None:
        if isinstance(tensors, torch.Tensor):
            if tensors.is_contiguous():
                self._reduce_tensor(tensors.view(-1), **kwargs)
            else:
                flat = tensors.reshape(-1).clone()
                self._reduce_tensor(flat, **kwargs)
                tensors.copy_(flat.view_as(tensors))
            return
        tensors = list(tensors)
        flat = torch.cat([t.reshape(-1) for t in tensors])
        self._reduce_tensor(flat, **kwargs)
        off = 0
        for t in tensors:
            t.copy_(flat[off: off + t.numel()].view_as(t))
            off += t.numel()


class LinearReducer(TensorReducer):
    def __init__(self, process_group=None, normalize: bool = True, weight_softmax_temperature: Optional[float] = None):
        super().__init__(process_group, weight_softmax_temperature)
        self.normalize = normalize and weight_softmax_temperature is None

    def _reduce_tensor(self, tensor, **kwargs):
        w = self._refine_weight(tensor.device, tensor.dtype, **kwargs)
        tensor.mul_(w)
        if self.normalize:
            div = w.clone().reshape(1)
            dist.all_reduce(div, group=self.process_group)
            if div.abs().item() < 1e-8:
                div.fill_(1.0)
            tensor.div_(div)
        dist.all_reduce(tensor, group=self.process_group)


def consensus_mask(delta: torch.Tensor, method: str, mask_dtype, group) -> torch.Tensor:
    if method == "sum":
        tot = delta.clone()
    elif method == "count":
        tot = delta.sign()
    else:
        raise RuntimeError(f"unknown consensus method {method!r}")
    dist.all_reduce(tot, group=group)
    majority = (tot >= 0).to(mask_dtype) * 2 - 1
    return delta.sign().to(mask_dtype) == majority


def get_consensus_mask_distributed(delta, method="sum", mask_dtype=None, process_group=None) -> torch.Tensor:
    """``consensus_mask`` under the reference's name and argument order."""
    return consensus_mask(delta, method, delta.dtype if mask_dtype is None else mask_dtype, process_group)


class GTAReducer(TensorReducer):
    def __init__(self, process_group=None, consensus_method: Optional[str] = None,
                 sparsification_method: Optional[str] = None, normalize: bool = True, density: float = 1.0,
                 int8_mask: bool = False, weight_softmax_temperature: Optional[float] = None):
        super().__init__(process_group, weight_softmax_temperature)
        self.consensus_method, self.sparsification_method = consensus_method, sparsification_method
        self.normalize, self.density, self.int8_mask = normalize, density, int8_mask

    def _reduce_tensor(self, tensor, **kwargs):
        if self.sparsification_method:
            tensor.copy_(sparsify(tensor, self.density, str(getattr(self.sparsification_method, "value",
                                                                       self.sparsification_method))))
        w = self._refine_weight(tensor.device, tensor.dtype, **kwargs)
        tensor.mul_(w)
        mask = None
        if self.consensus_method:
            mask = consensus_mask(tensor, self.consensus_method, torch.int8 if self.int8_mask else tensor.dtype,
                                  self.process_group)
            tensor.mul_(mask.to(tensor.dtype))
        if self.normalize:
            div = (mask.to(tensor.dtype) * w) if mask is not None else w.clone().reshape(1)
            dist.all_reduce(div, group=self.process_group)
            div = torch.where(div.abs() < 1e-8, torch.ones_like(div), div)
            tensor.div_(div)
        dist.all_reduce(tensor, group=self.process_group)


def build_reducer(gta_config, process_group, weight_softmax_temperature=None):
    if gta_config is None or gta_config.reducer is None:
        return None
    if gta_config.reducer == "linear":
        return LinearReducer(process_group, gta_config.normalize, weight_softmax_temperature)
    if gta_config.reducer == "gta":
        return GTAReducer(process_group, gta_config.consensus_method, gta_config.sparsification_method,
                          gta_config.normalize, gta_config.density, gta_config.int8_mask, weight_softmax_temperature)
    return None
