"""Data-parallel gradient averaging with flat buckets.

Parameters are packed, in reverse registration order (the order gradients become ready), into flat
buckets of ``bucket_cap_mb``; every ``param.grad`` is a view into its bucket, so a finished bucket
is all-reduced in place, on a communication stream, while the backward pass continues. Buckets
that never became complete (unused parameters) are reduced when the backward pass ends, so the
loop needs no ``find_unused_parameters`` probing pass.

On 2 to 8 GPUs of one NVSwitch domain all buckets are ranges of ONE symmetric buffer and each bucket is
reduced by this package's own kernel (csrc/comm.cu ``p2p_allreduce_kernel``: multimem.ld_reduce +
multimem.st through the switch, or two-shot peer loads) with the 1/world scaling folded in; elsewhere
(CPU/gloo, more ranks, mixed gradient dtypes) the buckets go through ``dist.all_reduce``.

Plays the role of ``torch.nn.parallel.DistributedDataParallel`` as applied by the ``parallel_mode``
/ ``auto_ddp`` optimisations of the reference (atorch/auto/opt_lib/parallel_mode_optimization.py:22-62).
"""
from __future__ import annotations

import contextlib
import os
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


class _Bucket:
    ALIGN = 64   # elements: a multiple of world * (16 bytes / element size) for every supported world size

    def __init__(self, params: List[nn.Parameter], device, dtype, storage: Optional[torch.Tensor] = None,
                 storage_offset: int = 0):
        self.params = params
        n = sum(p.numel() for p in params)
        self.padded = (n + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.offset = storage_offset
        if storage is not None:
            self.flat = storage[storage_offset: storage_offset + self.padded]
            self.flat.zero_()
        else:
            self.flat = torch.zeros(self.padded, dtype=dtype, device=device)
        self.views, off = [], 0
        for p in params:
            self.views.append(self.flat[off: off + p.numel()].view_as(p))
            off += p.numel()
        self.pending = len(params)
        self.launched = False


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, process_group: Optional[dist.ProcessGroup] = None,
                 bucket_cap_mb: float = 25.0, find_unused_parameters: bool = False, broadcast_buffers: bool = True,
                 sync_module_states: bool = True, gradient_predivide: bool = True, comm_blocks: int = 32,
                 param_filter=None):
        super().__init__()
        self.module = module
        self.comm_blocks = comm_blocks      # CTAs one bucket all-reduce may occupy beside the backward kernels
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.require_backward_grad_sync = True
        self.broadcast_buffers = broadcast_buffers
        # ``param_filter(name, param) -> bool`` restricts this reducer to some of the parameters (the
        # mixture-of-experts wrapper runs one reducer per group of ranks that replicate them)
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        if param_filter is not None:
            named = [(n, p) for n, p in named if param_filter(n, p)]
        params = [p for _, p in named]
        self._own = {id(p) for p in params}
        self.device = params[0].device if params else torch.device("cpu")
        self.comm_stream = torch.cuda.Stream(self.device) if (self.device.type == "cuda" and self.world > 1) else None
        if sync_module_states and self.world > 1:
            src = dist.get_global_rank(process_group, 0) if process_group is not None else 0
            own_params = [p for p in module.parameters() if param_filter is None or id(p) in self._own]
            bufs = list(module.buffers()) if (param_filter is None or broadcast_buffers) else []
            for t in own_params + bufs:
                dist.broadcast(t.data, src=src, group=process_group)
        self.buckets: List[_Bucket] = []
        cap = int(bucket_cap_mb * 1024 * 1024)
        groups, cur, cur_bytes, cur_dtype = [], [], 0, None
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > cap or p.dtype != cur_dtype):
                groups.append((cur, cur_dtype))
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_dtype = p.dtype
        if cur:
            groups.append((cur, cur_dtype))
        self.symm = self._make_symmetric(groups)
        off = 0
        for ps, dt in groups:
            b = _Bucket(ps, self.device, dt, None if self.symm is None else self.symm.tensor, off)
            off += b.padded
            self.buckets.append(b)
        self._bucket_of = {}
        for b in self.buckets:
            for p, v in zip(b.params, b.views):
                self._bucket_of[id(p)] = b
                p.register_post_accumulate_grad_hook(self._make_hook(b))
        self._cb_queued = False

    def _make_symmetric(self, groups):
        """One symmetric buffer for all buckets, when this package's all-reduce kernel can run."""
        dtypes = {dt for _, dt in groups}
        if not (self.device.type == "cuda" and 1 < self.world <= 8 and len(dtypes) == 1
                and next(iter(dtypes)) in (torch.float32, torch.bfloat16)
                and os.environ.get("ATB_FUSED_COMM", "1") != "0"):
            return None
        from . import symm

        if not symm.available():
            return None
        total = sum((sum(p.numel() for p in ps) + _Bucket.ALIGN - 1) // _Bucket.ALIGN * _Bucket.ALIGN
                    for ps, _ in groups)
        try:
            return symm.SymmetricBuffer(total, next(iter(dtypes)), self.group, self.device)
        except Exception as e:   # no symmetric memory on this system: NCCL buckets
            import logging

            logging.getLogger("atorch.logger").warning("DDP: own all-reduce kernel disabled: %s", e)
            return None

    def _attach_views(self):
        if self.symm is not None:
            self.symm.wait_peers_done()     # peers may still read last step's buckets
        for b in self.buckets:
            if all(p.grad is None for p in b.params):      # the usual case after zero_grad(): one fill per bucket
                b.flat.zero_()
                for p, v in zip(b.params, b.views):
                    p.grad = v
                continue
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
            if self.symm is not None:
                self.symm.all_reduce_(scale=1.0 / self.world, numel=bucket.padded, offset=bucket.offset,
                                      max_blocks=self.comm_blocks)
            else:
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
