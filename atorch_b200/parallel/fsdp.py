"""Fully sharded data parallel (ZeRO-3 / ZeRO-2 / hybrid shard) engine.

Design (one process per GPU, written for 180 GB HBM3e parts):

* The model is cut into *units* (each module of a wrap class, plus a root unit for what is left).
  A unit's parameters live back to back in one flat buffer with 16-byte aligned starts, padded to
  a multiple of the shard group size.
* Each rank owns ``1/W`` of every flat buffer. All shards of all units sit in ONE global fp32
  *master* buffer, one global fp32 *gradient* buffer and (under mixed precision) one global
  low-precision *working* buffer, so the optimizer step is a single fused kernel over the whole
  model (``FusedShardedOptimizer``) and gradient-norm clipping is one reduction.
* Compute uses the unit's full low-precision buffer: all-gathered from the working shards on a
  communication stream one unit ahead of the compute stream (forward and backward prefetch) and
  freed after use; with one rank the working buffer *is* the full buffer and nothing is copied.
* A unit runs as one autograd node: its backward re-gathers the parameters, optionally recomputes
  the forward (activation checkpointing per unit), back-propagates with weight gradients
  accumulated by the GEMM epilogues straight into the unit's flat gradient buffer
  (``param.main_grad``), then reduce-scatters that buffer into the fp32 gradient shard.
* Works on CPU with the gloo backend as well (used by the tests; no streams there).

Behavioural counterpart in the reference: the ``fsdp`` / ``zero2`` optimisations wrapping torch FSDP
(atorch/auto/opt_lib/zero_optimization.py:287-502, options ``atorch_wrap_cls``,
``atorch_size_based_min_num_params``, ``atorch_ignored_cls``, mixed precision folded in from
``amp_native`` at atorch/auto/model_context.py:598-608, HYBRID_SHARD when both ``zero`` and
``data`` groups exist :453-471).
"""
from __future__ import annotations

import contextlib
import math
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils._pytree import tree_flatten, tree_unflatten

from .. import ops
from ..utils.checkpoint import checkpoint_pass, new_pass_token

_RS_PREWAIT = os.environ.get("ATB_RS_PREWAIT", "0") == "1"   # see _reduce_grads_fused
ALIGN = 8  # elements: 16 bytes in bf16, so every parameter can be a TMA operand


def _align_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


@dataclass
class ShardingConfig:
    process_group: Optional[dist.ProcessGroup] = None      # shard group (None = default group)
    replica_group: Optional[dist.ProcessGroup] = None      # hybrid shard: all-reduce across replicas
    param_dtype: Optional[torch.dtype] = None               # compute dtype (None = keep fp32)
    reduce_dtype: Optional[torch.dtype] = None               # gradient reduce dtype (None = param dtype)
    reshard_after_forward: bool = True                       # False = ZeRO-2 style (keep params gathered)
    forward_prefetch: bool = True
    backward_prefetch: bool = True
    sync_module_states: bool = False
    param_init_fn: Optional[Callable[[nn.Module], None]] = None
    device: Optional[torch.device] = None
    checkpoint_units: bool = False                           # recompute each non-root unit in backward
    fused_comm: Optional[bool] = None                        # own collectives over peer memory instead of NCCL
    #                                                          (None: on when available, unless ATB_FUSED_COMM=0)
    optimizer_in_backward: bool = False                      # AdamW of a unit right after its reduce-scatter
    comm_blocks: int = 32                                    # CTAs a fused collective may occupy
    prefetch_depth: int = 2                                  # units gathered ahead of the computing one
    autocast: bool = True                                    # run forward under autocast(param_dtype)


class FlatUnit:
    """Parameters of one sharding unit laid out in a flat buffer."""

    def __init__(self, engine: "FSDPEngine", name: str, module: nn.Module,
                 params: List[Tuple[str, nn.Parameter]], is_root: bool):
        self.engine, self.name, self.module, self.is_root = engine, name, module, is_root
        self.param_names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.shapes = [tuple(p.shape) for p in self.params]
        self.numels = [p.numel() for p in self.params]
        self.offsets: List[int] = []
        off = 0
        for n in self.numels:
            self.offsets.append(off)
            off = _align_up(off + n, ALIGN)
        self.numel = off
        W = engine.world
        self.padded_numel = _align_up(max(off, 1), W * ALIGN)
        self.shard_numel = self.padded_numel // W
        self.shard_offset = 0           # start inside the engine's global shard buffers
        self.full: Optional[torch.Tensor] = None
        self.full_grad: Optional[torch.Tensor] = None
        self.gathered = False
        self.gather_event = None
        self.fresh = True               # next gradient accumulation overwrites instead of adding
        self.checkpoint = False
        self.orig_forward = None
        self.has_trainable = any(p.requires_grad for p in self.params)
        self._zero_ranges: Optional[List[Tuple[int, int]]] = None

    # flat <-> parameter views -----------------------------------------------------------------
    def views(self, flat: torch.Tensor) -> List[torch.Tensor]:
        return [flat[o: o + n].view(s) for o, n, s in zip(self.offsets, self.numels, self.shapes)]

    def shard_range(self, rank: Optional[int] = None) -> Tuple[int, int]:
        r = self.engine.rank if rank is None else rank
        return r * self.shard_numel, (r + 1) * self.shard_numel

    def uncovered_ranges(self, covered: Sequence[bool]) -> List[Tuple[int, int]]:
        """Ranges of the flat buffer NOT inside a parameter flagged in ``covered``: alignment gaps,
        the tail padding and the parameters left out. Adjacent ranges are merged."""
        out: List[Tuple[int, int]] = []
        pos = 0
        for o, n, c in zip(self.offsets, self.numels, covered):
            if c:
                if o > pos:
                    out.append((pos, o))
                pos = o + n
        if pos < self.padded_numel:
            out.append((pos, self.padded_numel))
        return out

    def trainable_shard_segments(self) -> List[Tuple[int, int]]:
        """Maximal runs of trainable parameters inside this rank's shard, as (start, end) offsets in the
        shard. A run includes the alignment gaps between its parameters (and the tail padding when the
        last parameter is trainable): their master values and gradients are zero, so an optimizer
        update leaves them zero. Frozen parameters are never part of a run."""
        lo, hi = self.shard_range()
        segs: List[Tuple[int, int]] = []
        bounds = list(self.offsets[1:]) + [self.padded_numel]
        for o, nxt, p in zip(self.offsets, bounds, self.params):
            if not p.requires_grad:
                continue
            s, e = max(o, lo), min(nxt, hi)
            if e <= s:
                continue
            if segs and segs[-1][1] == s - lo:
                segs[-1] = (segs[-1][0], e - lo)
            else:
                segs.append((s - lo, e - lo))
        return segs

    def param_shard_slices(self) -> List[Tuple[int, int, int]]:
        """For each parameter: (start in this rank's shard, length, start inside the parameter)."""
        lo, hi = self.shard_range()
        out = []
        for o, n in zip(self.offsets, self.numels):
            s, e = max(o, lo), min(o + n, hi)
            out.append((s - lo, max(e - s, 0), max(s - o, 0)) if e > s else (0, 0, 0))
        return out


def _flatten_io(obj) -> Tuple[list, Any]:
    return tree_flatten(obj)


class _UnitFn(torch.autograd.Function):
    """Forward/backward of one non-root unit as a single autograd node."""

    @staticmethod
    def forward(ctx, unit: FlatUnit, spec, n_in: int, *flat):
        eng = unit.engine
        ctx.unit, ctx.spec = unit, spec
        ctx.n_extra = len(flat) - n_in
        flat = list(flat[:n_in])
        ctx.tensor_idx = [i for i, t in enumerate(flat) if isinstance(t, torch.Tensor)]
        ctx.proto = [None if isinstance(t, torch.Tensor) else t for t in flat]
        ctx.autocast = (torch.is_autocast_enabled(eng.device.type), torch.get_autocast_dtype(eng.device.type)) \
            if hasattr(torch, "get_autocast_dtype") else (False, None)
        eng._pre_forward(unit, will_backward=True)
        if unit.checkpoint:
            ctx.save_for_backward(*[flat[i] for i in ctx.tensor_idx])
            ctx.token = new_pass_token()
            with torch.no_grad(), checkpoint_pass(ctx.token, False):
                args, kwargs = tree_unflatten(flat, spec)
                out = unit.orig_forward(*args, **kwargs)
            ctx.inner = None
        else:
            inner_in = []
            for i in ctx.tensor_idx:
                d = flat[i].detach()
                d.requires_grad_(flat[i].requires_grad)
                flat[i] = d
                inner_in.append(d)
            with torch.enable_grad():
                args, kwargs = tree_unflatten(flat, spec)
                out = unit.orig_forward(*args, **kwargs)
            ctx.inner = (inner_in, out)
        eng._post_forward(unit)
        out_flat, out_spec = tree_flatten(out)
        ctx.out_spec = out_spec
        ctx.out_tensor_idx = [i for i, t in enumerate(out_flat) if isinstance(t, torch.Tensor)]
        unit._last_out_spec = (out_spec, [None if isinstance(t, torch.Tensor) else t for t in out_flat],
                               ctx.out_tensor_idx)
        outs = tuple(out_flat[i].detach() if ctx.inner is not None else out_flat[i] for i in ctx.out_tensor_idx)
        nondiff = [o for o in outs if not o.is_floating_point()]
        if nondiff:
            ctx.mark_non_differentiable(*nondiff)
        return outs

    @staticmethod
    def backward(ctx, *gout):
        unit, eng = ctx.unit, ctx.unit.engine
        eng._pre_backward(unit)
        if ctx.inner is None:
            flat = list(ctx.proto)
            inner_in = []
            for i, t in zip(ctx.tensor_idx, ctx.saved_tensors):
                d = t.detach()
                d.requires_grad_(t.requires_grad)
                flat[i] = d
                inner_in.append(d)
            ac_on, ac_dt = ctx.autocast
            cm = torch.autocast(eng.device.type, dtype=ac_dt) if ac_on else contextlib.nullcontext()
            with torch.enable_grad(), cm, checkpoint_pass(ctx.token, True):
                args, kwargs = tree_unflatten(flat, ctx.spec)
                out = unit.orig_forward(*args, **kwargs)
        else:
            inner_in, out = ctx.inner
            ctx.inner = None
        out_flat, _ = tree_flatten(out)
        outs = [out_flat[i] for i in ctx.out_tensor_idx]
        pairs = [(o, g) for o, g in zip(outs, gout) if g is not None and o.requires_grad]
        if pairs:
            torch.autograd.backward([p[0] for p in pairs], [p[1] for p in pairs])
        grads = [None] * len(ctx.proto)
        for i, d in zip(ctx.tensor_idx, inner_in):
            grads[i] = d.grad
        eng._post_backward(unit)
        return (None, None, None, *grads, *([None] * ctx.n_extra))


class FSDPEngine:
    """Owns the units, the global shard buffers, the streams and the schedule."""

    def __init__(self, module: nn.Module, unit_modules: Sequence[nn.Module], config: ShardingConfig,
                 ignored_params: Optional[Set[nn.Parameter]] = None):
        self.module, self.cfg = module, config
        self.group = config.process_group
        distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(self.group) if distributed else 1
        self.rank = dist.get_rank(self.group) if distributed else 0
        self.replicas = dist.get_world_size(config.replica_group) if (distributed and config.replica_group is not None) else 1
        dev = config.device
        if dev is None:
            dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(dev)
        self.on_cuda = self.device.type == "cuda"
        self.compute_dtype = config.param_dtype or torch.float32
        self.mixed = self.compute_dtype != torch.float32
        self.reduce_dtype = config.reduce_dtype or self.compute_dtype
        multi = self.on_cuda and self.world * self.replicas > 1
        # all-gathers and reduce-scatters run on streams of their own, so that the prefetch of the
        # next unit's parameters never queues behind the reduction of the previous unit's gradients
        self.ag_stream = torch.cuda.Stream(self.device) if multi else None
        self.rs_stream = torch.cuda.Stream(self.device) if multi else None
        self.opt_stream = None                # 1-rank optimizer-in-backward (see FusedShardedOptimizer)
        self._rs_group = None                 # second communicator for NCCL reduce-scatters (lazy)
        self.ignored = ignored_params or set()
        self.units: List[FlatUnit] = []
        self.exec_order: List[FlatUnit] = []
        self._bwd_pending = False
        self._final_cb_queued = False
        self.grad_shard: Optional[torch.Tensor] = None
        self._shard_params: Optional[List[Tuple[str, nn.Parameter]]] = None
        self.training_step = 0
        self.local_sgd = None            # set by local_sgd.sharded.attach_local_sgd
        self.accumulation_boundary = True  # False while micro-batches of one step are still being accumulated
        self._fp32_accum = False
        self._build(unit_modules)

    # ------------------------------------------------------------------------------------ build
    def _build(self, unit_modules: Sequence[nn.Module]) -> None:
        unit_set = {id(m): m for m in unit_modules if m is not self.module}
        names = {id(m): n for n, m in self.module.named_modules()}
        # own parameters of a module subtree, stopping at nested unit boundaries
        def own_params(root: nn.Module, prefix: str) -> List[Tuple[str, nn.Parameter]]:
            res = []
            stack = [(prefix, root)]
            while stack:
                pre, m = stack.pop(0)
                for n, p in m._parameters.items():
                    if p is not None:
                        res.append((pre + n, p))
                for n, c in m._modules.items():
                    if c is None or (id(c) in unit_set and c is not root):
                        continue
                    stack.append((pre + n + ".", c))
            return res

        self._materialize_meta(unit_set)
        for m in self.module.modules():
            for n in getattr(m, "_atb_direct_grad_params", ()):
                try:
                    m.get_parameter(n)._atb_direct_grad = True
                except AttributeError:
                    pass
        seen: Set[int] = set()
        ordered = [m for _, m in self.module.named_modules() if id(m) in unit_set]
        plan = [(names[id(m)], m, False) for m in ordered] + [("", self.module, True)]
        for name, m, is_root in plan:
            ps = []
            for fq, p in own_params(m, name + "." if name else ""):
                if id(p) in seen or p in self.ignored:
                    continue
                seen.add(id(p))
                ps.append((fq, p))
            if not ps and not is_root:
                continue
            u = FlatUnit(self, name, m, ps, is_root)
            u.checkpoint = self.cfg.checkpoint_units and not is_root
            self.units.append(u)
        off = 0
        for u in self.units:
            u.shard_offset = off
            off += u.shard_numel
        self.total_shard = off
        dev = self.device
        self.master = torch.zeros(off, dtype=torch.float32, device=dev)
        self.lp_shard = torch.zeros(off, dtype=self.compute_dtype, device=dev) if self.mixed else None
        for u in self.units:
            self._init_unit_storage(u)
        self._non_root_units = [x for x in self.units if not x.is_root]
        self._non_root_index = {id(x): i for i, x in enumerate(self._non_root_units)}
        self._wrap_unit_forwards()
        self._setup_fused_comm()

    N_GRAD_BUFFERS = 3

    def _setup_fused_comm(self) -> None:
        """Own collectives over NVLink peer memory (parallel/symm.py, csrc/comm.cu):

        * the low-precision working shards live in ONE symmetric buffer; a unit is all-gathered by the
          copy engines straight out of the peers' shards (no SM, no NCCL kernel next to the GEMMs);
        * gradients are written into symmetric buffers - ``N_GRAD_BUFFERS`` rotating ones of the largest
          non-root unit plus one for the root unit, which stays live for the whole backward - and
          reduce-scattered by a kernel that reads the peers' slices (or lets the switch add them) and
          writes the fp32 gradient shard or runs AdamW in the same pass."""
        self.fused = False
        self._fused_opt = None
        want = self.cfg.fused_comm
        if want is None:
            want = os.environ.get("ATB_FUSED_COMM", "1") != "0"
        if not (want and self.on_cuda and 1 < self.world <= 8 and self.replicas == 1
                and self.compute_dtype == torch.bfloat16):
            return
        from . import symm

        if not symm.available():
            return
        try:
            non_root = [u.padded_numel for u in self.units if not u.is_root and u.has_trainable]
            self._gbufs = [symm.SymmetricBuffer(max(non_root), self.compute_dtype, self.group, self.device)
                           for _ in range(self.N_GRAD_BUFFERS)] if non_root else []
            root = self.units[-1]
            self._root_gbuf = symm.SymmetricBuffer(root.padded_numel, self.compute_dtype, self.group, self.device) \
                if root.has_trainable else None
            self._lp_symm = symm.SymmetricBuffer(self.total_shard, self.compute_dtype, self.group, self.device)
        except Exception as e:   # symmetric memory unavailable on this system: keep the NCCL path
            import logging

            logging.getLogger("atorch.logger").warning("fused collectives disabled: %s", e)
            return
        self._lp_symm.tensor.copy_(self.lp_shard)
        self.lp_shard = self._lp_symm.tensor
        self._gbuf_events = [None] * self.N_GRAD_BUFFERS
        self._gbuf_rr = 0
        self._param_seq = self._lp_symm.signal(symm.CH_READY)     # this rank's parameters are in place
        self._ready_waited = 0
        self.fused = True

    def _params_changed(self) -> None:
        """The working shards were rewritten on the current stream (optimizer step, state-dict load)."""
        if self.fused:
            from . import symm

            self._param_seq = self._lp_symm.signal(symm.CH_READY)

    def _materialize_meta(self, unit_set) -> None:
        """Give meta-device parameters real storage on the target device, module by module."""
        def init_one(m: nn.Module):
            if not any(p.is_meta for p in m._parameters.values() if p is not None) and \
               not any(b.is_meta for b in m._buffers.values() if b is not None):
                return
            m.to_empty(device=self.device, recurse=False)
            if self.cfg.param_init_fn is not None:
                self.cfg.param_init_fn(m)
            elif hasattr(self.module, "_init_weights"):
                if hasattr(m, "reset_parameters"):
                    m.reset_parameters()
                self.module._init_weights(m)
            elif hasattr(m, "reset_parameters"):
                m.reset_parameters()
            else:
                raise RuntimeError(f"cannot initialise meta module {type(m).__name__}: pass param_init_fn")
        if any(p.is_meta for p in self.module.parameters()):
            for m in self.module.modules():
                init_one(m)

    def _init_unit_storage(self, u: FlatUnit) -> None:
        dev = self.device
        flat = torch.zeros(u.padded_numel, dtype=torch.float32, device=dev)
        for v, p in zip(u.views(flat), u.params):
            v.copy_(p.detach().to(device=dev, dtype=torch.float32))
        if self.cfg.sync_module_states and self.world > 1:
            dist.broadcast(flat, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                           group=self.group)
        lo, hi = u.shard_range()
        so = u.shard_offset
        self.master[so: so + u.shard_numel].copy_(flat[lo:hi])
        if self.mixed:
            self.lp_shard[so: so + u.shard_numel].copy_(flat[lo:hi])
        if self.world == 1:
            src = self.lp_shard if self.mixed else self.master
            u.full = src[so: so + u.padded_numel]
            u.gathered = True
        else:
            u.full = flat.to(self.compute_dtype) if self.mixed else flat
            u.gathered = True
        for v, p in zip(u.views(u.full), u.params):
            p.data = v
            p._atb_unit = u
        if self.world > 1:
            self._free_full(u)
        del flat

    def _wrap_unit_forwards(self) -> None:
        for u in self.units:
            if u.is_root:
                continue
            u.orig_forward = u.module.forward
            u.module._atb_fsdp_unit = u
            u.module.forward = self._make_unit_forward(u)

    def _make_unit_forward(self, u: FlatUnit):
        def unit_forward(*args, **kwargs):
            flat, spec = tree_flatten((args, kwargs))
            needs_graph = torch.is_grad_enabled() and (
                u.has_trainable or any(isinstance(t, torch.Tensor) and t.requires_grad for t in flat))
            if not needs_graph:
                self._pre_forward(u)
                out = u.orig_forward(*args, **kwargs)
                self._post_forward(u)
                return out
            # the node must be differentiable even if no input requires grad (first unit of a model):
            # an extra scalar that requires grad rides along after the real arguments
            extra = []
            if not any(isinstance(t, torch.Tensor) and t.requires_grad for t in flat):
                extra = [torch.zeros((), device=self.device, requires_grad=True)]
            outs = _UnitFn.apply(u, spec, len(flat), *flat, *extra)
            out_spec, proto, tidx = u._last_out_spec
            out_flat = list(proto)
            for i, t in zip(tidx, outs):
                out_flat[i] = t
            return tree_unflatten(out_flat, out_spec)
        return unit_forward

    # ------------------------------------------------------------------------- gather / release
    def _alloc_full(self, u: FlatUnit) -> None:
        st = u.full.untyped_storage()
        nbytes = u.padded_numel * u.full.element_size()
        if st.size() != nbytes:
            st.resize_(nbytes)

    def _free_full(self, u: FlatUnit) -> None:
        if self.world == 1:
            return
        if u.gather_event is not None:            # a prefetch still in flight writes into this storage
            torch.cuda.current_stream(self.device).wait_event(u.gather_event)
        u.full.untyped_storage().resize_(0)
        u.gathered = False
        u.gather_event = None

    def _shard_src(self, u: FlatUnit) -> torch.Tensor:
        src = self.lp_shard if self.mixed else self.master
        return src[u.shard_offset: u.shard_offset + u.shard_numel]

    def _unshard(self, u: FlatUnit) -> None:
        if u.gathered:
            return
        self._alloc_full(u)
        src = self._shard_src(u)
        if self.fused:
            from . import symm

            cur = torch.cuda.current_stream(self.device)
            self.ag_stream.wait_stream(cur)       # earlier users of the buffer's memory come first
            with torch.cuda.stream(self.ag_stream):
                if self._ready_waited != self._param_seq:      # once per parameter version
                    self._lp_symm.wait(symm.CH_READY, self._param_seq)
                    self._ready_waited = self._param_seq
                self._lp_symm.copy_engine_all_gather(u.full, u.shard_offset, u.shard_numel)
                ev = torch.cuda.Event()
                ev.record(self.ag_stream)
            u.gather_event = ev
        elif self.ag_stream is not None:
            cur = torch.cuda.current_stream(self.device)
            self.ag_stream.wait_stream(cur)
            with torch.cuda.stream(self.ag_stream):
                dist.all_gather_into_tensor(u.full, src, group=self.group)
                ev = torch.cuda.Event()
                ev.record(self.ag_stream)
            u.gather_event = ev
        else:
            dist.all_gather_into_tensor(u.full, src, group=self.group)
        u.gathered = True

    def _wait_unshard(self, u: FlatUnit) -> None:
        if u.gather_event is not None:
            torch.cuda.current_stream(self.device).wait_event(u.gather_event)
            u.gather_event = None

    # ------------------------------------------------------------------------------- schedule
    def _pre_forward(self, u: FlatUnit, will_backward: bool = False) -> None:
        """``will_backward``: this forward is an autograd node, so the unit goes on the list the backward prefetch
        walks in reverse (grad mode cannot tell: it is off inside an autograd function's forward)."""
        self._unshard(u)
        self._wait_unshard(u)
        if will_backward or torch.is_grad_enabled():
            self.exec_order.append(u)
        if self.cfg.forward_prefetch and self.world > 1:
            for nxt in self._next_in_order(u):
                self._unshard(nxt)

    def _next_in_order(self, u: FlatUnit) -> List[FlatUnit]:
        """The ``prefetch_depth`` units that follow ``u`` in the forward pass."""
        us = self._non_root_units
        i = self._non_root_index.get(id(u))
        if i is None:
            return []
        return us[i + 1: i + 1 + max(1, self.cfg.prefetch_depth)]

    def _post_forward(self, u: FlatUnit) -> None:
        if self.cfg.reshard_after_forward and not u.is_root:
            self._free_full(u)

    def _direct_grads(self) -> bool:
        """One rank, no replicas: the unit gradient buffers ARE slices of the global gradient buffer
        (compute dtype), nothing is reduced or copied. Accumulating over micro-batches switches the
        engine to an fp32 gradient shard (see ``_switch_to_fp32_accumulation``)."""
        return self.world == 1 and self.replicas == 1 and not self._fp32_accum

    def _switch_to_fp32_accumulation(self) -> None:
        if self._fp32_accum:
            return
        self._fp32_accum = True
        if self.grad_shard is not None and self.grad_shard.dtype != torch.float32:
            self.grad_shard = self.grad_shard.float()

    def _first_write_ok(self) -> bool:
        """Kernels that write a parameter gradient can overwrite on first touch (no zero fill) only when
        the kernel path is certain: CUDA, library loaded, bf16 compute."""
        from .. import _lib

        return self.on_cuda and self.compute_dtype == torch.bfloat16 and _lib.have_kernels()

    def _alloc_grads(self, u: FlatUnit) -> None:
        if u.full_grad is not None or not u.has_trainable:
            return
        if self._direct_grads() and not u.fresh:
            self._switch_to_fp32_accumulation()       # a second micro-batch: accumulate in fp32 from now on
        if self._direct_grads():
            self._ensure_grad_shard()
            u.full_grad = self.grad_shard[u.shard_offset: u.shard_offset + u.padded_numel]
        elif self.fused:
            if u.is_root:
                buf, u._gbuf_idx = self._root_gbuf, -1
            else:
                idx = self._gbuf_rr % self.N_GRAD_BUFFERS
                self._gbuf_rr += 1
                buf, u._gbuf_idx = self._gbufs[idx], idx
                if self._gbuf_events[idx] is not None:   # this rank's previous reduce-scatter out of this buffer
                    torch.cuda.current_stream(self.device).wait_event(self._gbuf_events[idx])
                    self._gbuf_events[idx] = None
            buf.wait_peers_done()                        # ... and the peers' reads of it (bounded wait kernel)
            u._gbuf = buf
            u.full_grad = buf.tensor[: u.padded_numel]
        else:
            u.full_grad = torch.empty(u.padded_numel, dtype=self.compute_dtype, device=self.device)
        first_ok = self._first_write_ok()
        if not first_ok:
            u.full_grad.zero_()
        else:
            # only parameters whose gradient kernel overwrites on first touch may stay uninitialised:
            # alignment gaps, tail padding, frozen parameters and every other parameter start at zero
            # (the whole buffer is reduced, normed and fed to the optimizer)
            if u._zero_ranges is None:
                u._zero_ranges = u.uncovered_ranges(
                    [p.requires_grad and getattr(p, "_atb_direct_grad", False) for p in u.params])
            for s0, e0 in u._zero_ranges:
                u.full_grad[s0:e0].zero_()
        for v, p in zip(u.views(u.full_grad), u.params):
            if p.requires_grad:
                if first_ok and getattr(p, "_atb_direct_grad", False):
                    p._atb_first = True               # the writing kernel overwrites instead of accumulating
                p.grad = v
                p.main_grad = v

    def _pre_backward(self, u: FlatUnit) -> None:
        self._unshard(u)
        self._wait_unshard(u)
        self._alloc_grads(u)
        if self.cfg.backward_prefetch and self.world > 1 and u in self.exec_order:
            i = self.exec_order.index(u)
            for j in range(i - 1, max(i - 1 - max(1, self.cfg.prefetch_depth), -1), -1):
                self._unshard(self.exec_order[j])

    def _post_backward(self, u: FlatUnit) -> None:
        self._reduce_grads(u)
        if not u.is_root:
            self._free_full(u)

    def _ensure_grad_shard(self) -> None:
        if self.grad_shard is None:
            dt = self.compute_dtype if (self.world == 1 and self.replicas == 1 and not self._fp32_accum) \
                else torch.float32
            self.grad_shard = torch.zeros(self.total_shard, dtype=dt, device=self.device)

    def _reduce_grads(self, u: FlatUnit) -> None:
        g = u.full_grad
        if g is None:
            return
        if self._fused_opt is not None:
            self._fused_opt.guard(u)
        for v, p in zip(u.views(g), u.params):
            if getattr(p, "_atb_first", False):       # no kernel wrote this gradient in this backward
                v.zero_()
                p._atb_first = False
            p.grad = None
            if hasattr(p, "main_grad"):
                del p.main_grad
        u.full_grad = None
        if self._direct_grads():
            opt = self._fused_opt
            if opt is not None and opt.in_backward_ready(u):
                opt.local_unit_step(u)                # AdamW of this unit overlaps the rest of the backward
            u.fresh = False                           # gradients already sit in the global buffer
            return
        self._ensure_grad_shard()
        dst = self.grad_shard[u.shard_offset: u.shard_offset + u.shard_numel]
        skip_rep = self.local_sgd is not None and self.local_sgd.skip_replica_reduce()
        scale = 1.0 / (self.world * (1 if skip_rep else self.replicas))
        if self.world == 1 and self.replicas == 1:
            if u.fresh:
                dst.copy_(g)
            else:
                dst.add_(g)
            u.fresh = False
            return
        if self.fused:
            self._reduce_grads_fused(u, dst, scale)
            return
        rd = g if g.dtype == self.reduce_dtype else g.to(self.reduce_dtype)
        out = torch.empty(u.shard_numel, dtype=self.reduce_dtype, device=self.device)
        if self.rs_stream is not None:
            cur = torch.cuda.current_stream(self.device)
            self.rs_stream.wait_stream(cur)
            cm = torch.cuda.stream(self.rs_stream)
        else:
            cm = contextlib.nullcontext()
        with cm:
            if self.world > 1:
                dist.reduce_scatter_tensor(out, rd, op=dist.ReduceOp.SUM, group=self._reduce_group())
            else:
                out.copy_(rd)
            if self.replicas > 1 and not (self.local_sgd is not None and self.local_sgd.skip_replica_reduce()):
                dist.all_reduce(out, group=self.cfg.replica_group)
            if u.fresh:
                dst.copy_(out)
                dst.mul_(scale)
            else:
                dst.add_(out, alpha=scale)
        if self.rs_stream is not None:
            rd.record_stream(self.rs_stream)
            out.record_stream(self.rs_stream)
            g.record_stream(self.rs_stream)
        u.fresh = False

    def _reduce_group(self):
        """NCCL path: reduce-scatters use a communicator of their own (same ranks as the shard group), so
        that they do not serialise with the all-gather prefetch inside one communicator's stream."""
        if not self.on_cuda or os.environ.get("ATB_NCCL_SPLIT_STREAMS", "1") == "0":
            return self.group
        if self._rs_group is None:
            ranks = dist.get_process_group_ranks(self.group if self.group is not None else dist.group.WORLD)
            self._rs_group = dist.new_group(ranks)
        return self._rs_group

    def _reduce_grads_fused(self, u: FlatUnit, dst: torch.Tensor, scale: float) -> None:
        """One kernel per unit on the reduction stream: the peers' gradient slices are summed over
        NVLink (peer loads in registers, or multimem.ld_reduce in the switch) and land in the fp32
        gradient shard - or, with ``optimizer_in_backward``, go straight through the AdamW update into
        master / moments / working shard."""
        cur = torch.cuda.current_stream(self.device)
        self.rs_stream.wait_stream(cur)
        buf = u._gbuf
        with torch.cuda.stream(self.rs_stream):
            opt = self._fused_opt
            if opt is not None and opt.in_backward_ready(u):
                opt.fused_unit_step(buf, u, u.shard_offset)
            else:
                if _RS_PREWAIT:
                    # One warp waits until every rank's gradients of this unit are complete; only then does the
                    # multi-CTA kernel start. Its own arrival wait would otherwise keep its CTAs resident (and the
                    # persistent GEMM CTAs that share their SMs slow) for as long as the slowest rank is behind.
                    from . import symm

                    buf.wait(symm.CH_READY, buf.signal(symm.CH_READY))
                buf.reduce_scatter_into(dst, scale=scale, accumulate=not u.fresh, numel=u.padded_numel,
                                        max_blocks=self.cfg.comm_blocks)
            if u._gbuf_idx >= 0:
                ev = torch.cuda.Event()
                ev.record(self.rs_stream)
                self._gbuf_events[u._gbuf_idx] = ev
        u.fresh = False

    # ------------------------------------------------------------------------------ root hooks
    def root_pre_forward(self) -> None:
        self.exec_order = []
        root = self.units[-1]
        self._unshard(root)
        self._wait_unshard(root)
        if self.world > 1 and self.cfg.forward_prefetch:
            for first in self._non_root_units[: max(1, self.cfg.prefetch_depth)]:
                self._unshard(first)
        if torch.is_grad_enabled():
            self._alloc_grads(root)

    def root_post_forward(self, out):
        if not torch.is_grad_enabled():
            return out
        flat, spec = tree_flatten(out)
        hooked = False
        for t in flat:
            if isinstance(t, torch.Tensor) and t.requires_grad:
                t.register_hook(self._on_backward_start)
                hooked = True
        self._final_cb_queued = False
        self._bwd_pending = hooked
        return out

    def _on_backward_start(self, grad):
        if not self._final_cb_queued:
            self._final_cb_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._final_callback)
        return grad

    def _final_callback(self) -> None:
        root = self.units[-1]
        self._reduce_grads(root)
        for u in self.units:
            if u.full_grad is not None:     # unit whose backward node never ran (unused outputs)
                self._reduce_grads(u)
            if not u.is_root and self.world > 1 and u.gathered:
                self._free_full(u)
        if self.rs_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.rs_stream)
        if self.opt_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.opt_stream)
        self._bwd_pending = False
        self._final_cb_queued = False

    # ----------------------------------------------------------------------- optimizer support
    def zero_grad(self) -> None:
        for u in self.units:
            u.fresh = True

    def finalize_grads(self) -> torch.Tensor:
        """fp32 gradient shard with never-touched units zeroed; call before an optimizer step."""
        self._ensure_grad_shard()
        for u in self.units:
            if u.fresh:
                self.grad_shard[u.shard_offset: u.shard_offset + u.shard_numel].zero_()
                u.fresh = False
        return self.grad_shard

    def shard_parameters(self) -> List[Tuple[str, nn.Parameter]]:
        """fp32 views of this rank's part of every original parameter (possibly empty), with their
        names: what a sharded optimizer updates. ``.grad`` is attached by ``attach_shard_grads``."""
        if self._shard_params is None:
            res = []
            for u in self.units:
                ms = self.master[u.shard_offset: u.shard_offset + u.shard_numel]
                for name, p, (s, n, _) in zip(u.param_names, u.params, u.param_shard_slices()):
                    sp = nn.Parameter(ms[s: s + n], requires_grad=p.requires_grad)
                    sp._atb_fqn = name
                    res.append((name, sp))
            self._shard_params = res
        return self._shard_params

    def attach_shard_grads(self) -> None:
        g = self.finalize_grads()
        if g.dtype != torch.float32:                  # generic optimizers want gradients in the parameter dtype
            self._switch_to_fp32_accumulation()
            g = self.grad_shard
        it = iter(self.shard_parameters())
        for u in self.units:
            gs = g[u.shard_offset: u.shard_offset + u.shard_numel]
            for (s, n, _) in u.param_shard_slices():
                _, sp = next(it)
                sp.grad = gs[s: s + n] if sp.requires_grad else None

    def sync_working_copy(self) -> None:
        """After an optimizer updated the fp32 master: refresh the low-precision working shards."""
        if self.mixed:
            self.lp_shard.copy_(self.master)
        self.invalidate_gathered()

    def invalidate_gathered(self) -> None:
        """Parameters changed (optimizer step, state-dict load): gathered copies are stale."""
        self._params_changed()
        if self.world > 1:
            for u in self.units:
                if u.gathered:
                    self._free_full(u)

    def grad_norm(self, norm_type: float = 2.0) -> torch.Tensor:
        g = self.finalize_grads()
        if norm_type == math.inf:
            n = g.abs().max()
            if self.world > 1:
                dist.all_reduce(n, op=dist.ReduceOp.MAX, group=self.group)
            return n
        if norm_type == 2.0:
            s = ops.sum_squares(g)
        else:
            s = g.abs().pow(norm_type).sum()
        if self.world > 1:
            dist.all_reduce(s, group=self.group)
        return s.pow(1.0 / norm_type)

    def clip_grad_norm_(self, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
        total = self.grad_norm(norm_type)
        coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
        self.grad_shard.mul_(coef)
        return total

    # -------------------------------------------------------------------------- state dict I/O
    def gather_unit_master(self, u: FlatUnit) -> torch.Tensor:
        ms = self.master[u.shard_offset: u.shard_offset + u.shard_numel]
        if self.world == 1:
            return ms
        full = torch.empty(u.padded_numel, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(full, ms.contiguous(), group=self.group)
        return full

    def full_state_dict(self, rank0_only: bool = False, cpu: bool = True) -> Dict[str, torch.Tensor]:
        sd: Dict[str, torch.Tensor] = {}
        keep = (not rank0_only) or self.rank == 0
        for u in self.units:
            full = self.gather_unit_master(u)
            if keep:
                for name, v in zip(u.param_names, u.views(full)):
                    sd[name] = v.detach().cpu().clone() if cpu else v.detach().clone()
        if keep:
            for n, b in self.module.named_buffers():
                sd[n] = b.detach().cpu().clone() if cpu else b.detach().clone()
        return sd

    def load_full_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> None:
        for u in self.units:
            lo, hi = u.shard_range()
            ms = self.master[u.shard_offset: u.shard_offset + u.shard_numel]
            for name, (s, n, ps) in zip(u.param_names, u.param_shard_slices()):
                if name not in sd:
                    if strict:
                        raise KeyError(name)
                    continue
                if n:
                    ms[s: s + n].copy_(sd[name].reshape(-1)[ps: ps + n].to(torch.float32))
        self.sync_working_copy()
        if self.local_sgd is not None:
            self.local_sgd.reset_baseline()       # new weights: the next pseudo-gradient starts from them
        for n, b in self.module.named_buffers():
            if n in sd:
                b.copy_(sd[n])

    def summon_full_params(self):
        """Context manager: all parameters gathered (read access to full values)."""
        eng = self

        @contextlib.contextmanager
        def cm():
            for u in eng.units:
                eng._unshard(u)
                eng._wait_unshard(u)
            try:
                yield
            finally:
                for u in eng.units:
                    if not u.is_root or eng.world > 1:
                        eng._free_full(u)
        return cm()


def _resolve_wrap_modules(module: nn.Module, wrap_cls, min_num_params: Optional[int]) -> List[nn.Module]:
    if wrap_cls:
        classes, names = [], set()
        for c in (wrap_cls if isinstance(wrap_cls, (tuple, list, set)) else (wrap_cls,)):
            if isinstance(c, str):
                names.add(c)
            else:
                classes.append(c)
        classes = tuple(classes)
        return [m for m in module.modules()
                if m is not module and ((classes and isinstance(m, classes)) or type(m).__name__ in names)]
    if min_num_params:
        # size based: post-order, wrap a subtree once its not-yet-wrapped parameters reach the limit
        chosen: List[nn.Module] = []
        def visit(m: nn.Module) -> int:
            rest = sum(p.numel() for p in m._parameters.values() if p is not None)
            for c in m._modules.values():
                if c is not None:
                    rest += visit(c)
            if m is not module and rest >= min_num_params:
                chosen.append(m)
                return 0
            return rest
        visit(module)
        return chosen
    return []


class FSDP(nn.Module):
    """Sharded data-parallel wrapper around ``module``.

    ``parameters()`` / ``named_parameters()`` yield this rank's fp32 shard views under the original
    parameter names (what an optimizer should be built on); ``forward`` runs the wrapped module with
    parameters gathered unit by unit. ``wrap_cls`` may hold classes or class names.
    """

    def __init__(self, module: nn.Module, wrap_cls=None, min_num_params: Optional[int] = None,
                 ignored_cls=None, config: Optional[ShardingConfig] = None, **cfg_kwargs):
        super().__init__()
        config = config or ShardingConfig(**cfg_kwargs)
        self.module = module
        ignored: Set[nn.Parameter] = set()
        if ignored_cls:
            for m in module.modules():
                if isinstance(m, tuple(ignored_cls)):
                    ignored.update(m.parameters())
        units = _resolve_wrap_modules(module, wrap_cls, min_num_params)
        self.engine = FSDPEngine(module, units, config, ignored)
        dev = self.engine.device
        for m in module.modules():
            for n, b in list(m._buffers.items()):
                if b is not None and b.device != dev and not b.is_meta:
                    m._buffers[n] = b.to(dev)
        for p in ignored:
            p.data = p.data.to(dev)

    def forward(self, *args, **kwargs):
        eng = self.engine
        eng.root_pre_forward()
        use_ac = eng.mixed and eng.cfg.autocast
        cm = torch.autocast(eng.device.type, dtype=eng.compute_dtype) if use_ac else contextlib.nullcontext()
        with cm:
            out = self.module(*args, **kwargs)
        return eng.root_post_forward(out)

    # optimizer-facing parameter view ------------------------------------------------------------
    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        for n, p in self.engine.shard_parameters():
            yield (prefix + ("." if prefix else "") + n, p)

    def parameters(self, recurse: bool = True):
        for _, p in self.named_parameters():
            yield p

    def zero_grad(self, set_to_none: bool = True):
        self.engine.zero_grad()

    @contextlib.contextmanager
    def no_sync(self):
        """Gradients are reduce-scattered every micro-batch and accumulated in the fp32 shard, so
        there is nothing to postpone; provided for loop compatibility."""
        yield

    def clip_grad_norm_(self, max_norm: float, norm_type: float = 2.0):
        return self.engine.clip_grad_norm_(max_norm, norm_type)

    def state_dict(self, *args, rank0_only: bool = False, **kwargs):
        return self.engine.full_state_dict(rank0_only=rank0_only)

    def load_state_dict(self, sd, strict: bool = True, **kwargs):
        self.engine.load_full_state_dict(sd, strict)

    def summon_full_params(self):
        return self.engine.summon_full_params()


class ShardedOptimizer:
    """Adapter that lets any ``torch.optim.Optimizer`` built on ``FSDP.parameters()`` drive the
    engine: attaches gradient shards before the step, refreshes the working copy after it."""

    def __init__(self, optimizer: torch.optim.Optimizer, engine: FSDPEngine):
        self.optimizer, self.engine = optimizer, engine

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def state(self):
        return self.optimizer.state

    def step(self, closure=None):
        self.engine.attach_shard_grads()
        r = self.optimizer.step(closure) if closure is not None else self.optimizer.step()
        self.engine.sync_working_copy()
        if self.engine.local_sgd is not None:
            self.engine.local_sgd.after_optimizer_step()
        return r

    def zero_grad(self, set_to_none: bool = True):
        self.engine.zero_grad()

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, sd):
        self.optimizer.load_state_dict(sd)

    def __getattr__(self, k):
        return getattr(self.optimizer, k)


class FusedShardedOptimizer:
    """AdamW / AGD over the engine's global flat shards in one kernel launch per step
    (csrc/optim.cu). Moment buffers are allocated lazily as fp32 twins of the master buffer."""

    def __init__(self, engine: FSDPEngine, kind: str = "adamw", lr: float = 1e-3, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01, delta: float = 1e-5, clip: Optional[float] = None,
                 weight_decouple: bool = True, fixed_decay: bool = False, max_grad_norm: Optional[float] = None):
        assert kind in ("adamw", "adam", "agd")
        self.engine, self.kind = engine, kind
        self.defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, delta=delta)
        self.param_groups = [dict(self.defaults, params=[p for _, p in engine.shard_parameters()])]
        self.clip, self.weight_decouple, self.fixed_decay = clip, weight_decouple, fixed_decay
        self.max_grad_norm = max_grad_norm
        self.exp_avg: Optional[torch.Tensor] = None
        self.exp_avg_sq: Optional[torch.Tensor] = None
        self.step_count = 0
        self.state: Dict = {}
        self._stepped: Set[int] = set()          # ids of the units already updated in this backward pass
        self._segs: Dict = {}
        if engine.cfg.optimizer_in_backward and max_grad_norm is None and engine.mixed and (
                (getattr(engine, "fused", False) and kind == "adamw")
                or (engine.world == 1 and engine.replicas == 1 and engine.on_cuda)):
            engine._fused_opt = self

    # ----------------------------------------------------------------- optimizer inside the backward
    def in_backward_ready(self, u) -> bool:
        """May unit ``u`` be updated right after its gradients are complete? Only on the boundary
        micro-batch of a step whose gradients were not accumulated, and only for units without frozen
        parameters (the per-unit kernels update the whole shard of the unit)."""
        eng = self.engine
        self.guard(u)
        return (eng.accumulation_boundary and u.fresh and u.has_trainable
                and all(p.requires_grad for p in u.params))

    def guard(self, u) -> None:
        if id(u) in self._stepped:
            raise RuntimeError(
                "optimizer_in_backward: a second backward pass reached a unit that was already updated in "
                "this step. With gradient accumulation call set_gradient_accumulation_boundary(False) "
                "before every micro-batch but the last one of a step.")

    def set_gradient_accumulation_boundary(self, flag: bool) -> None:
        self.engine.accumulation_boundary = bool(flag)

    def fused_unit_step(self, buf, u, so: int) -> None:
        """Reduce-scatter + AdamW of one unit inside the backward pass (called on the reduction stream)."""
        self._ensure_state()
        eng, pg = self.engine, self.param_groups[0]
        n = u.shard_numel
        b1, b2 = pg["betas"]
        lp = eng.lp_shard[so: so + n] if eng.mixed else None
        buf.reduce_scatter_adamw(eng.master[so: so + n], self.exp_avg[so: so + n], self.exp_avg_sq[so: so + n], lp,
                                 pg["lr"], b1, b2, pg["eps"], pg["weight_decay"], self.step_count + 1,
                                 grad_scale=1.0 / eng.world, numel=u.padded_numel, max_blocks=eng.cfg.comm_blocks)
        self._stepped.add(id(u))

    def local_unit_step(self, u) -> None:
        """One rank: the update of unit ``u`` runs on a side stream while the backward pass goes on. The
        memory-bound optimizer kernel shares the SMs with the compute-bound GEMMs (its grid is capped so
        that GEMM CTAs still fit beside it), which hides most of its 28 bytes per parameter."""
        self._ensure_state()
        eng = self.engine
        if eng.opt_stream is None:
            eng.opt_stream = torch.cuda.Stream(eng.device)
        cur = torch.cuda.current_stream(eng.device)
        eng.opt_stream.wait_stream(cur)
        sl = slice(u.shard_offset, u.shard_offset + u.shard_numel)
        with torch.cuda.stream(eng.opt_stream):
            self._update(sl, eng.grad_shard, self.step_count + 1, None, max_blocks=2 * 148)
        self._stepped.add(id(u))

    # -------------------------------------------------------------------------------- ordinary step
    def _update(self, sl: slice, g: torch.Tensor, step: int, scale_t, max_blocks: int = 0) -> None:
        eng, pg = self.engine, self.param_groups[0]
        b1, b2 = pg["betas"]
        lp = eng.lp_shard[sl] if eng.lp_shard is not None else None
        if self.kind == "agd":
            ops.agd_step(eng.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], g[sl], lp, pg["lr"], b1, b2,
                         pg["delta"], pg["weight_decay"], step, grad_scale_tensor=scale_t,
                         clip=self.clip, decouple=self.weight_decouple, fixed_decay=self.fixed_decay)
        else:
            ops.adamw_step(eng.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], g[sl], lp, pg["lr"], b1, b2,
                           pg["eps"], pg["weight_decay"], step, grad_scale_tensor=scale_t,
                           adamw_mode=self.kind == "adamw", max_blocks=max_blocks)

    def _segments(self, skip: Optional[Set[int]] = None) -> List[Tuple[int, int]]:
        """Ranges of the global shard buffers that the step updates: everything when all parameters
        train (one launch), otherwise the runs of trainable parameters - frozen parameters get neither
        an update nor weight decay. Units whose id is in ``skip`` are left out."""
        key = frozenset(skip) if skip else None
        if key not in self._segs:
            segs: List[Tuple[int, int]] = []
            for u in self.engine.units:
                if skip and id(u) in skip:
                    continue
                for s0, e0 in u.trainable_shard_segments():
                    a, b = u.shard_offset + s0, u.shard_offset + e0
                    if segs and segs[-1][1] == a:
                        segs[-1] = (segs[-1][0], b)
                    else:
                        segs.append((a, b))
            self._segs[key] = segs
        return self._segs[key]

    def _ensure_state(self):
        if self.exp_avg is None:
            self.exp_avg = torch.zeros_like(self.engine.master)
            self.exp_avg_sq = torch.zeros_like(self.engine.master)

    def zero_grad(self, set_to_none: bool = True):
        self.engine.zero_grad()

    def step(self, closure=None):
        loss = closure() if closure is not None else None
        eng = self.engine
        stepped, self._stepped = self._stepped, set()
        if stepped:
            # these units were updated during the backward pass; wait for those kernels
            cur = torch.cuda.current_stream(eng.device)
            for st in (eng.rs_stream, eng.opt_stream):
                if st is not None:
                    cur.wait_stream(st)
        todo = self._segments(stepped)
        self._ensure_state()
        self.step_count += 1
        if todo:
            g = eng.finalize_grads()
            scale_t = None
            if self.max_grad_norm is not None and self.max_grad_norm > 0:
                total = eng.grad_norm(2.0)
                scale_t = (self.max_grad_norm / (total + 1e-6)).clamp(max=1.0).float().reshape(1)
                self.last_grad_norm = total
            for s0, e0 in todo:
                self._update(slice(s0, e0), g, self.step_count, scale_t)
        eng.invalidate_gathered()
        if eng.local_sgd is not None:
            eng.local_sgd.after_optimizer_step()
        return loss

    def state_dict(self):
        self._ensure_state()
        return {"kind": self.kind, "step": self.step_count, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd):
        self._ensure_state()
        self.step_count = int(sd["step"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        for g, s in zip(self.param_groups, sd.get("param_groups", [])):
            g.update(s)
