"""Selective activation offloading inside a checkpointed region.

Instead of recomputing everything, the outputs of chosen operators (by name, e.g. ``mm.default``,
and by occurrence index) are copied to pinned host memory on a side stream during the forward and
copied back in the backward; all other tensors are recomputed. Implemented with saved-tensor hooks
around the module forward: a saved tensor produced by a selected op call is replaced by a handle
to its host copy.
(Reference: atorch/auto/opt_lib/selective_offloading_checkpoint.py:68-252,
``OffloadOpManagerArgs(name, index_to_offload, index_to_hold, index_to_hold_layer)``.)
"""
from __future__ import annotations

import functools
from typing import Dict, List, Optional

import torch
from torch.utils._python_dispatch import TorchDispatchMode


class OffloadOpManagerArgs:
    def __init__(self, name: str = "mm.default", index_to_offload: Optional[List[int]] = None,
                 index_to_hold: Optional[List[int]] = None, index_to_hold_layer: Optional[List[int]] = None):
        self.name, self.index_to_offload = name, list(index_to_offload or [])
        self.index_to_hold, self.index_to_hold_layer = list(index_to_hold or []), list(index_to_hold_layer or [])


class _Tracker(TorchDispatchMode):
    """Records the data pointers of the outputs of selected op calls."""

    def __init__(self, specs: List[OffloadOpManagerArgs]):
        super().__init__()
        self.specs = specs
        self.counts: Dict[str, int] = {}
        self.selected = set()

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        name = str(func).replace("aten.", "")
        for sp in self.specs:
            if name.endswith(sp.name):
                i = self.counts.get(sp.name, 0)
                self.counts[sp.name] = i + 1
                if i in sp.index_to_offload and isinstance(out, torch.Tensor):
                    self.selected.add(out.data_ptr())
        return out


def offload_forward(inner_forward, offload_config):
    """Wrap a module forward: saved tensors coming from the selected ops live on the host between
    forward and backward."""
    specs = []
    for item in (offload_config.get("offload_args") or []):
        if isinstance(item, OffloadOpManagerArgs):
            specs.append(item)
        else:
            specs.append(OffloadOpManagerArgs(*item))
    stream_holder = {}

    @functools.wraps(inner_forward)
    def fwd(*a, **k):
        if not torch.is_grad_enabled():
            return inner_forward(*a, **k)
        tracker = _Tracker(specs)
        cuda = torch.cuda.is_available()
        if cuda and "s" not in stream_holder:
            stream_holder["s"] = torch.cuda.Stream()

        def pack(t):
            if t.data_ptr() not in tracker.selected or not t.is_cuda:
                return ("keep", t)
            s = stream_holder["s"]
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
                host.copy_(t, non_blocking=True)
            t.record_stream(s)
            return ("host", host, t.device)

        def unpack(h):
            if h[0] == "keep":
                return h[1]
            stream_holder["s"].synchronize()
            return h[1].to(h[2], non_blocking=True)
        with torch.autograd.graph.saved_tensors_hooks(pack, unpack), tracker:
            return inner_forward(*a, **k)
    return fwd
