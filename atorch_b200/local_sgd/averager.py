"""Local SGD for replicated (DDP-style) training: ``OuterOptimPeriodicModelAverager`` and
``StatefulPostLocalSGDOptimizer``.

Every replica trains alone for H inner steps; then the *pseudo-gradient* ``last_synced - param`` is
averaged over the replicas and an outer optimizer (typically SGD lr 0.7, momentum 0.9, Nesterov)
steps the last synchronised weights, which are written back into the parameters:

    g = last_synced - p;  [anomaly: g = 0];  g = reduce(g);  [clip];  outer step on last_synced;  p <- last_synced

Here all of that state is ONE flat fp32 buffer on the GPU (the reference keeps ``last_synced`` per
parameter on the CPU and copies per parameter, atorch/local_sgd/DDP/outer_optim_model_averager.py:87):
the pseudo-gradient of the whole model is one subtraction, one all-reduce and, for SGD/Nesterov,
one fused update kernel (``ops.outer_sgd_step``, csrc/optim.cu). Other outer optimizer classes run
as ordinary torch optimizers on the flat ``last_synced`` parameter.

On 2 to 8 GPUs of one NVSwitch domain, plain SGD/Nesterov without reducer, anomaly skipping or clipping
takes ONE kernel for the whole outer step (csrc/comm.cu ``p2p_allreduce_nesterov_kernel``): the
replicas' parameters sit in a symmetric buffer, every rank owns 1/W of the outer state (synchronised
weights and momentum), reduces the mean of its slice over the peers (peer loads or multimem.ld_reduce),
applies the Nesterov update and hands the new weights to every replica - no pseudo-gradient tensor,
no separate all-reduce, and the outer state costs 1/W of the memory.
(Reference: atorch/local_sgd/DDP/outer_optim_model_averager.py:17-194,
stateful_post_localSGD_optimizer.py:6-20.)
"""
from __future__ import annotations

import time
from typing import Dict, Iterable, List, Optional, Union

import torch
import torch.distributed as dist

from .. import ops
from .anomaly import OnlineDynamicEWMA
from .configs import GTAConfig, LocalSGDConfig, OuterOptimizerConfig
from .reducers import build_reducer


def get_params_to_average(params) -> List[torch.nn.Parameter]:
    out = []
    for p in params:
        if isinstance(p, dict):
            out.extend(q for q in p["params"] if q.grad is not None or q.requires_grad)
        elif isinstance(p, torch.nn.Parameter) or isinstance(p, torch.Tensor):
            out.append(p)
    return out


class OuterOptimPeriodicModelAverager:
    def __init__(self, process_group=None, local_sgd_config: Optional[LocalSGDConfig] = None,
                 gta_config: Optional[GTAConfig] = None, outer_optim_config: Optional[OuterOptimizerConfig] = None):
        self.process_group = process_group if process_group is not None else dist.group.WORLD
        self.local_sgd_config = local_sgd_config or LocalSGDConfig()
        self.gta_config = gta_config or GTAConfig()
        self.outer_optim_config = outer_optim_config or OuterOptimizerConfig()
        c = self.local_sgd_config
        self.step = 0
        self.warmup_steps, self.local_sgd_sync_interval = c.local_sgd_warmup_steps, c.local_sgd_sync_interval
        self.clip_pseudo_grad, self.skip_anomaly = c.clip_pseudo_grad, c.skip_anomaly
        self.pseudo_gradnorm_reduce = c.pseudo_gradnorm_reduce
        temp = c.weight_softmax_temperature
        if self.pseudo_gradnorm_reduce and temp is None:
            temp = 1.0
        self.reducer = build_reducer(self.gta_config, self.process_group, temp)
        self.last_synced: Optional[torch.nn.Parameter] = None     # flat fp32
        self.momentum_buf: Optional[torch.Tensor] = None
        self.outer_optimizer: Optional[torch.optim.Optimizer] = None
        self._fused_sgd: Optional[dict] = None
        self._pending_outer_sd = None
        self._offsets: List[int] = []
        self.anomaly_detectors: Optional[List[OnlineDynamicEWMA]] = None
        self.outer_steps = 0
        self._symm = None                  # symmetric parameter buffer of the one-kernel outer step
        self._slice = None                 # (lo, hi) of this rank's part of the outer state
        # asynchronous mode: the decision to synchronise is taken on wall-clock time (mean over the ranks)
        self.use_async, self.sync_time = c.use_async, c.local_sgd_sync_time
        self.min_total_global_steps = c.min_total_global_steps
        self.use_step_weight, self.step_weight_ratio = c.use_step_weight, c.step_weight_ratio
        self.cpu_offload = c.cpu_offload
        self.last_sync_timestamp: Optional[float] = None
        self.last_total_global_step = 0
        self._step_at_last_sync = 0
        self._clock = time.time      # replaceable in tests

    # ------------------------------------------------------------------------------- state
    def state_dict(self) -> Dict:
        sd: Dict = {"step": self.step}
        if self.outer_optimizer is not None:
            sd["outer_optimizer"] = torch.utils._pytree.tree_map(
                lambda x: x.cpu() if isinstance(x, torch.Tensor) else x, self.outer_optimizer.state_dict())
        elif self._fused_sgd is not None and self.momentum_buf is not None:
            sd["outer_optimizer"] = {"fused_sgd": dict(self._fused_sgd),
                                     "momentum_buffer": self._full_state(self.momentum_buf).cpu(),
                                     "outer_steps": self.outer_steps}
        if self.anomaly_detectors is not None:
            sd["anomaly_detectors"] = [d.state_dict() for d in self.anomaly_detectors]
        return sd

    def load_state_dict(self, sd: Dict) -> None:
        self.step = sd["step"]
        if "outer_optimizer" in sd:
            if self.last_synced is None:
                self._pending_outer_sd = sd["outer_optimizer"]
            else:
                self._load_outer(sd["outer_optimizer"])
        if "anomaly_detectors" in sd and self.anomaly_detectors is not None:
            for d, s in zip(self.anomaly_detectors, sd["anomaly_detectors"]):
                d.load_state_dict(s)

    def _full_state(self, t: torch.Tensor) -> torch.Tensor:
        """Outer-state tensor over the whole model (all-gathered when it is sharded 1/W per rank)."""
        if self._slice is None:
            return t
        world = dist.get_world_size(self.process_group)
        full = torch.empty(t.numel() * world, dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(full, t.contiguous(), group=self.process_group)
        return full[: self._numel]

    def _load_outer(self, osd) -> None:
        if "fused_sgd" in osd:
            mb = osd["momentum_buffer"]
            if self._slice is not None:
                pad = torch.zeros(self._symm.numel, dtype=mb.dtype)
                pad[: mb.numel()] = mb
                mb = pad[self._slice[0]: self._slice[1]]
            self.momentum_buf.copy_(mb)
            self.outer_steps = int(osd.get("outer_steps", 1))
        elif self.outer_optimizer is not None:
            self.outer_optimizer.load_state_dict(osd)

    # ------------------------------------------------------------------------------- set-up
    def _initialize(self, params: List[torch.nn.Parameter]) -> None:
        dev = params[0].device
        self._offsets, off = [], 0
        for p in params:
            self._offsets.append(off)
            off += p.numel()
        flat = torch.cat([p.detach().reshape(-1).float() for p in params])
        self._numel = flat.numel()
        cls, kw = self.outer_optim_config.outer_optim_class, dict(self.outer_optim_config.outer_optim_kwargs)
        plain_sgd = cls is torch.optim.SGD and not kw.get("dampening") and not kw.get("weight_decay") \
            and not kw.get("maximize")
        if plain_sgd and self._one_kernel_possible(dev):
            flat = self._setup_one_kernel(flat, dev)       # this rank's slice of the synchronised weights
        self.last_synced = torch.nn.Parameter(flat)
        if plain_sgd:
            self._fused_sgd = dict(lr=kw.get("lr", 1e-3), momentum=kw.get("momentum", 0.0),
                                   nesterov=bool(kw.get("nesterov", False)))
            self.momentum_buf = torch.zeros_like(flat)
        elif cls is not None:
            self.outer_optimizer = cls([self.last_synced], **kw)
        if self._pending_outer_sd is not None:
            self._load_outer(self._pending_outer_sd)
            self._pending_outer_sd = None
        if self.skip_anomaly:
            c = self.local_sgd_config
            self.anomaly_detectors = [OnlineDynamicEWMA(c.ewma_alpha, c.ewma_warmup_steps, c.ewma_threshold)
                                      for _ in params]

    def _one_kernel_possible(self, dev) -> bool:
        import os

        if dev.type != "cuda" or self.reducer is not None or self.skip_anomaly or self.pseudo_gradnorm_reduce \
                or self.clip_pseudo_grad is not None or os.environ.get("ATB_FUSED_COMM", "1") == "0" \
                or self.cpu_offload or (self.use_async and self.use_step_weight):
            return False
        from ..parallel import symm

        return symm.available() and 1 < dist.get_world_size(self.process_group) <= 8

    def _setup_one_kernel(self, flat: torch.Tensor, dev) -> torch.Tensor:
        from ..parallel import symm

        world, rank = dist.get_world_size(self.process_group), dist.get_rank(self.process_group)
        n = (flat.numel() + 4 * world - 1) // (4 * world) * (4 * world)
        try:
            self._symm = symm.SymmetricBuffer(n, torch.float32, self.process_group, dev)
        except Exception:
            self._symm = None
            return flat
        sl = n // world
        self._slice = (rank * sl, (rank + 1) * sl)
        padded = torch.zeros(n, dtype=torch.float32, device=dev)
        padded[: flat.numel()] = flat
        return padded[self._slice[0]: self._slice[1]].clone()

    def _all_reduce_scalar(self, v: float) -> float:
        dev = "cuda" if dist.get_backend(self.process_group) == "nccl" else "cpu"
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, group=self.process_group)
        return float(t.item())

    def should_sync(self) -> bool:
        """Step mode: every ``local_sgd_sync_interval`` steps after the warm-up. Asynchronous mode
        (``use_async``): when at least ``local_sgd_sync_time`` seconds of wall-clock time (mean of the ranks'
        clocks, so that every rank decides alike) have passed since the last synchronisation AND the replicas
        together have made at least ``min_total_global_steps`` steps since then; the first call after the
        warm-up synchronises and starts the clock. The small all-reduces of this test run every step on
        every rank. (Reference: atorch/local_sgd/FSDP/core/_runtime_utils.py:37-83.)"""
        if not self.use_async:
            return self.step >= self.warmup_steps and \
                (self.step - self.warmup_steps) % self.local_sgd_sync_interval == 0
        if self.step < self.warmup_steps:
            self.last_total_global_step = self._all_reduce_scalar(float(self.step))
            return False
        world = dist.get_world_size(self.process_group)
        now = self._all_reduce_scalar(self._clock() / world)
        if self.last_sync_timestamp is None:
            self.last_total_global_step = self._all_reduce_scalar(float(self.step))
            self.last_sync_timestamp = now
            return True
        if now - self.last_sync_timestamp < self.sync_time:
            return False
        total = self._all_reduce_scalar(float(self.step))
        self.last_sync_timestamp = now
        if total - self.last_total_global_step < self.min_total_global_steps:
            return False
        self.last_total_global_step = total
        return True

    def _step_weight(self, world: int) -> float:
        """Share of this replica in the steps made since the last synchronisation (asynchronous mode with
        ``use_step_weight``), else the plain ``1 / world``."""
        if not (self.use_async and self.use_step_weight):
            return 1.0 / world
        mine = float(self.step - self._step_at_last_sync)
        total = self._all_reduce_scalar(mine)
        return mine / total if total > 0 else 1.0 / world

    def _outer_state_to(self, device) -> None:
        """Moves the synchronised weights and the outer optimizer's tensors (CPU offload between outer steps)."""
        if self.last_synced is not None and self.last_synced.device != torch.device(device):
            self.last_synced.data = self.last_synced.data.to(device, non_blocking=True)
        if self.momentum_buf is not None and self.momentum_buf.device != torch.device(device):
            self.momentum_buf = self.momentum_buf.to(device, non_blocking=True)
        if self.outer_optimizer is not None:
            for st in self.outer_optimizer.state.values():
                for k, v in st.items():
                    if isinstance(v, torch.Tensor):
                        st[k] = v.to(device, non_blocking=True)

    # --------------------------------------------------------------------------------- step
    @torch.no_grad()
    def average_parameters(self, params: Union[Iterable[torch.nn.Parameter], Iterable[Dict]]) -> None:
        plain_average = self.outer_optim_config.outer_optim_class is None and self.reducer is None
        plist = None
        if not plain_average and self.last_synced is None:
            plist = get_params_to_average(params)
            self._initialize(plist)
        if self.should_sync():
            plist = plist if plist is not None else get_params_to_average(params)
            world = dist.get_world_size(self.process_group)
            if plain_average:
                flat = torch.cat([p.detach().reshape(-1).float() for p in plist])
                flat.mul_(self._step_weight(world))
                dist.all_reduce(flat, group=self.process_group)
                self._write_back(plist, flat)
            else:
                if self.cpu_offload and self._symm is None:
                    self._outer_state_to(plist[0].device)
                self._outer_step(plist, world)
                if self.cpu_offload and self._symm is None and plist[0].device.type != "cpu":
                    self._outer_state_to("cpu")
            self._step_at_last_sync = self.step
        self.step += 1

    def _write_back(self, plist, flat) -> None:
        for p, off in zip(plist, self._offsets or self._running_offsets(plist)):
            p.copy_(flat[off: off + p.numel()].view_as(p))

    @staticmethod
    def _running_offsets(plist):
        offs, off = [], 0
        for p in plist:
            offs.append(off)
            off += p.numel()
        return offs

    def _outer_step_one_kernel(self, plist) -> None:
        buf, f = self._symm, self._fused_sgd
        buf.wait_peers_done()                      # peers may still pull the previous result out of this buffer
        off = 0
        for p in plist:                            # the replicas' current parameters, fp32, into the symmetric buffer
            buf.tensor[off: off + p.numel()].copy_(p.detach().reshape(-1))
            off += p.numel()
        if off < buf.numel:
            buf.tensor[off:].zero_()
        buf.allreduce_nesterov(self.last_synced.data, self.momentum_buf, f["lr"], f["momentum"], f["nesterov"],
                               self.outer_steps == 0 or f["momentum"] == 0.0)
        self.outer_steps += 1
        self._write_back(plist, buf.tensor)        # every replica's buffer now holds the new weights

    def _outer_step(self, plist, world) -> None:
        if self._symm is not None:
            return self._outer_step_one_kernel(plist)
        cur = torch.cat([p.detach().reshape(-1).float() for p in plist])
        pg = self.last_synced.data - cur
        weight_kw = {}
        if self.skip_anomaly or self.pseudo_gradnorm_reduce:
            norms = [torch.linalg.vector_norm(pg[o: o + p.numel()]) for p, o in zip(plist, self._offsets)]
            total_norm = torch.linalg.vector_norm(torch.stack(norms))
            if self.skip_anomaly:
                for i, (p, o) in enumerate(zip(plist, self._offsets)):
                    if self.anomaly_detectors[i].is_outlier(norms[i]):
                        pg[o: o + p.numel()].zero_()
                        total_norm = total_norm + 1e6
                    else:
                        self.anomaly_detectors[i].update(norms[i])
            if self.pseudo_gradnorm_reduce:
                weight_kw["weight"] = -total_norm
        if self.reducer is None:
            pg.mul_(self._step_weight(world))
            dist.all_reduce(pg, group=self.process_group)
        else:
            if self.use_async and self.use_step_weight:
                weight_kw["step_weight"] = self._step_weight(world)
                weight_kw["step_weight_ratio"] = self.step_weight_ratio
            self.reducer.reduce_tensor(pg, **weight_kw)
        frozen = self.skip_anomaly and float(pg.abs().sum()) < 1e-6
        if not frozen:
            scale = 1.0
            if self.clip_pseudo_grad is not None and (self.outer_optimizer is not None or self._fused_sgd is not None):
                n = torch.linalg.vector_norm(pg)
                scale = float(torch.clamp(self.clip_pseudo_grad / (n + 1e-6), max=1.0))
            if self._fused_sgd is not None:
                f = self._fused_sgd
                ops.outer_sgd_step(self.last_synced.data, self.momentum_buf, pg, None, f["lr"], f["momentum"],
                                   f["nesterov"], self.outer_steps == 0 or f["momentum"] == 0.0, scale)
                self.outer_steps += 1
            elif self.outer_optimizer is not None:
                self.last_synced.grad = pg.mul_(scale) if scale != 1.0 else pg
                self.outer_optimizer.step()
                self.last_synced.grad = None
            else:
                self.last_synced.data.sub_(pg)
        self._write_back(plist, self.last_synced.data)


class StatefulPostLocalSGDOptimizer:
    """Runs the wrapped optimizer, then lets the averager decide whether this step synchronises.
    ``state_dict()["averager"]`` carries the averager state (step counter, outer optimizer)."""

    def __init__(self, optim, averager: OuterOptimPeriodicModelAverager):
        self.optim, self.averager = optim, averager

    @property
    def param_groups(self):
        return self.optim.param_groups

    @property
    def state(self):
        return self.optim.state

    def step(self, closure=None):
        r = self.optim.step(closure) if closure is not None else self.optim.step()
        self.averager.average_parameters(params=self.param_groups)
        return r

    def zero_grad(self, set_to_none: bool = True):
        self.optim.zero_grad(set_to_none=set_to_none)

    def add_param_group(self, g):
        self.optim.add_param_group(g)

    def state_dict(self):
        sd = self.optim.state_dict()
        sd["step"] = self.averager.step
        sd["averager"] = self.averager.state_dict()
        return sd

    def load_state_dict(self, sd):
        sd = dict(sd)
        asd = sd.pop("averager", None)
        step = sd.pop("step", None)
        self.optim.load_state_dict(sd)
        if asd is not None:
            self.averager.load_state_dict(asd)
        elif step is not None:
            self.averager.step = step


class PostLocalSGDState:
    """State of the gradient hook: gradients are all-reduced only until ``start_localSGD_iter``."""

    def __init__(self, process_group=None, subgroup=None, start_localSGD_iter: int = 0,
                 post_local_gradient_allreduce: bool = False):
        self.process_group, self.subgroup = process_group, subgroup
        self.start_localSGD_iter, self.post_local_gradient_allreduce = start_localSGD_iter, post_local_gradient_allreduce
        self.iter = 0

    def maybe_increase_iter(self):
        self.iter += 1


def post_localSGD_hook(ddp_model, state: PostLocalSGDState) -> None:
    """Install the post-local-SGD behaviour on this framework's DDP wrapper: bucket all-reduces run
    for the first ``start_localSGD_iter`` backward passes and are skipped afterwards."""
    orig_forward = ddp_model.forward

    def forward(*a, **k):
        if torch.is_grad_enabled():
            ddp_model.require_backward_grad_sync = state.iter < state.start_localSGD_iter
            state.maybe_increase_iter()
        return orig_forward(*a, **k)
    ddp_model.forward = forward
