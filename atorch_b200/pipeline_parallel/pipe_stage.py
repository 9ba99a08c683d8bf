"""One pipeline stage: a module chunk plus the mapping from received activations / batch fields to
its forward arguments, the per-micro-batch bookkeeping for backward, and its send/recv endpoints.

``input_output_mapping = {"default" | stage_id: (activation_mapping, batch_mapping)}`` with
``activation_mapping = [(forward_arg, activation_idx)]`` (None = all received activations,
positionally) and ``batch_mapping = [(forward_arg, batch_key_or_index)]`` (None = no batch data).
(Reference: atorch/pipeline_parallel/pipe_stage.py:24-343.)
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from ..communication.pipe_communicator import PipeCommunicator


def _as_tuple(x):
    if isinstance(x, torch.Tensor):
        return (x,)
    if isinstance(x, (tuple, list)):
        return tuple(t for t in x if isinstance(t, torch.Tensor))
    if isinstance(x, dict):
        return tuple(v for v in x.values() if isinstance(v, torch.Tensor))
    return tuple()


class PipeStage:
    def __init__(self, module: nn.Module, stage_id: int, num_stages: int, device, io_mapping: Optional[Dict],
                 comm: PipeCommunicator, stage_to_rank, my_rank: int):
        self.module, self.stage_id, self.num_stages, self.device = module, stage_id, num_stages, device
        self.comm, self.stage_to_rank, self.my_rank = comm, stage_to_rank, my_rank
        mapping = None
        if io_mapping is not None:
            mapping = io_mapping.get(stage_id, io_mapping.get(stage_id - num_stages, io_mapping.get("default")))
        self.activation_mapping, self.batch_mapping = mapping if mapping is not None else (None, None)
        self.is_first, self.is_last = stage_id == 0, stage_id == num_stages - 1
        self.fwd_cache: Dict[int, Any] = {}          # micro-batch -> (inputs requiring grad, outputs)
        self.ddp = module if hasattr(module, "no_sync") else None

    @property
    def prev_rank(self):
        return self.stage_to_rank(self.stage_id - 1)

    @property
    def next_rank(self):
        return self.stage_to_rank(self.stage_id + 1)

    # ------------------------------------------------------------------------------- forward
    def _build_kwargs(self, activations, batch):
        args, kwargs = [], {}
        if self.activation_mapping is None:
            args = list(activations)
        else:
            for name, idx in self.activation_mapping:
                kwargs[name] = activations[idx]
        if self.batch_mapping is not None and batch is not None:
            for name, key in self.batch_mapping:
                kwargs[name] = batch[key]
        return args, kwargs

    def forward_one_chunk(self, mb: int, activations, batch):
        acts = []
        for a in activations:
            a = a.detach()
            if a.is_floating_point():
                a.requires_grad_(True)
            acts.append(a)
        args, kwargs = self._build_kwargs(acts, batch)
        out = self.module(*args, **kwargs)
        self.fwd_cache[mb] = (acts, out)
        return out

    # ------------------------------------------------------------------------------ backward
    def backward_one_chunk(self, mb: int, loss: Optional[torch.Tensor], out_grads, last_microbatch: bool):
        acts, out = self.fwd_cache.pop(mb)
        ctx = self.ddp.no_sync() if (self.ddp is not None and not last_microbatch) else _null()
        with ctx:
            if loss is not None:
                loss.backward()
            else:
                outs = [o for o in _as_tuple(out) if o.requires_grad]
                torch.autograd.backward(outs, [g for g, o in zip(out_grads, _as_tuple(out)) if o.requires_grad])
        return [a.grad if a.grad is not None else torch.zeros_like(a) for a in acts if a.requires_grad]


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
