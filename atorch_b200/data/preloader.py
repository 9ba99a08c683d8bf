"""``GpuPreLoader``: overlap host->device copies (and optional post-processing) of the next batch
with the current step on a side CUDA stream; batches should come from pinned memory.
(Reference: atorch/data/preloader.py:8-194.)
"""
from __future__ import annotations

from typing import Callable, Iterable, Optional

import torch

from ..common.util_func import data_to_device


class GpuPreLoader:
    def __init__(self, dataloader: Iterable, device=None, post_processing: Optional[Callable] = None,
                 manual_preload: bool = False, mask=None):
        self.dataloader, self.post_processing, self.manual_preload = dataloader, post_processing, manual_preload
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.mask = mask
        self._it, self._next = None, None

    def __len__(self):
        return len(self.dataloader)

    def set_epoch(self, epoch: int) -> None:
        if hasattr(self.dataloader, "set_epoch"):
            self.dataloader.set_epoch(epoch)
        elif hasattr(getattr(self.dataloader, "sampler", None), "set_epoch"):
            self.dataloader.sampler.set_epoch(epoch)

    def _move(self, batch):
        if self.mask is not None and isinstance(batch, (list, tuple)):
            out = type(batch)(data_to_device(b, self.device) if m else b for b, m in zip(batch, self.mask))
        else:
            out = data_to_device(batch, self.device)
        return self.post_processing(out) if self.post_processing is not None else out

    def preload(self) -> None:
        try:
            batch = next(self._it)
        except StopIteration:
            self._next = None
            return
        if self.stream is None:
            self._next = self._move(batch)
            return
        with torch.cuda.stream(self.stream):
            self._next = self._move(batch)

    def __iter__(self):
        self._it = iter(self.dataloader)
        self.preload()
        return self

    def __next__(self):
        if self._next is None:
            raise StopIteration
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
            cur = torch.cuda.current_stream(self.device)
            for t in _tensors(self._next):
                t.record_stream(cur)
        batch = self._next
        if not self.manual_preload:
            self.preload()
        return batch


def _tensors(x):
    if isinstance(x, torch.Tensor):
        yield x
    elif isinstance(x, dict):
        for v in x.values():
            yield from _tensors(v)
    elif isinstance(x, (list, tuple)):
        for v in x:
            yield from _tensors(v)
