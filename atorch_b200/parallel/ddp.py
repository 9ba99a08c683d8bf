"""Data-parallel gradient averaging with flat buckets.

Parameters are packed, in reverse registration order (the order gradients become ready), into flat
buckets of ``bucket_cap_mb``; every ``param.grad`` is a view into its bucket, so a finished bucket
is all-reduced in place, on a communication stream, while the backward pass continues. Buckets
that never became complete (unused parameters) are reduced when the backward pass ends, so the
loop needs no ``find_unused_parameters`` probing pass.

Plays the role of ``torch.nn.parallel.DistributedDataParallel`` as applied by the ``parallel_mode``
/ ``auto_ddp`` optimisations of the reference (atorch/auto/opt_lib/parallel_mode_optimization.py:22-62).
"""
from __future__ import annotations

import contextlib
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


class _Bucket:
    def __init__(self, params: List[nn.Parameter], device, dtype):
        self.params = params
        n = sum(p.numel() for p in params)
        self.flat = torch.zeros(n, dtype=dtype, device=device)
        self.views, off = [], 0
        for p in params:
            self.views.append(self.flat[off: off + p.numel()].view_as(p))
            off += p.numel()
        self.pending = len(params)
        self.launched = False


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, process_group: Optional[dist.ProcessGroup] = None,
                 bucket_cap_mb: float = 25.0, find_unused_parameters: bool = False, broadcast_buffers: bool = True,
                 sync_module_states: bool = True, gradient_predivide: bool = True):
        super().__init__()
        self.module = module
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.require_backward_grad_sync = True
        self.broadcast_buffers = broadcast_buffers
        params = [p for p in module.parameters() if p.requires_grad]
        self.device = params[0].device if params else torch.device("cpu")
        self.comm_stream = torch.cuda.Stream(self.device) if (self.device.type == "cuda" and self.world > 1) else None
        if sync_module_states and self.world > 1:
            src = dist.get_global_rank(process_group, 0) if process_group is not None else 0
            for t in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(t.data, src=src, group=process_group)
        self.buckets: List[_Bucket] = []
        cap = int(bucket_cap_mb * 1024 * 1024)
        cur, cur_bytes, cur_dtype = [], 0, None
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > cap or p.dtype != cur_dtype):
                self.buckets.append(_Bucket(cur, self.device, cur_dtype))
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_dtype = p.dtype
        if cur:
            self.buckets.append(_Bucket(cur, self.device, cur_dtype))
        self._bucket_of = {}
        for b in self.buckets:
            for p, v in zip(b.params, b.views):
                self._bucket_of[id(p)] = b
                p.register_post_accumulate_grad_hook(self._make_hook(b))
        self._cb_queued = False

    def _attach_views(self):
        for b in self.buckets:
            for p, v in zip(b.params, b.views):
                if p.grad is None:
                    v.zero_()
                    p.grad = v
                elif p.grad.data_ptr() != v.data_ptr():
                    v.copy_(p.grad)
                    p.grad = v

    def _make_hook(self, bucket: _Bucket):
        def hook(param):
            if not self.require_backward_grad_sync or self.world == 1:
                return
            if not self._cb_queued:
                self._cb_queued = True
                torch.autograd.Variable._execution_engine.queue_callback(self._finish)
            bucket.pending -= 1
            if bucket.pending == 0:
                self._launch(bucket)
        return hook

    def _launch(self, bucket: _Bucket):
        bucket.launched = True
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            cm = torch.cuda.stream(self.comm_stream)
        else:
            cm = contextlib.nullcontext()
        with cm:
            bucket.flat.div_(self.world)
            dist.all_reduce(bucket.flat, group=self.group)

    def _finish(self):
        for b in self.buckets:
            if not b.launched:
                self._launch(b)
            b.pending, b.launched = len(b.params), False
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        self._cb_queued = False

    def forward(self, *args, **kwargs):
        if torch.is_grad_enabled():
            self._attach_views()
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        old = self.require_backward_grad_sync
        self.require_backward_grad_sync = False
        try:
            yield
        finally:
            self.require_backward_grad_sync = old

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, *a, **k):
        return self.module.load_state_dict(*a, **k)
