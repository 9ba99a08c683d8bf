"""Local SGD / EDiT on the sharded engine (hybrid shard: parameters sharded inside a ``zero`` group,
replicas across a ``data`` group).

After ``local_sgd_warmup_steps`` synchronous steps the gradient all-reduce across replicas is
switched off, every replica group trains on its own for ``local_sgd_sync_interval`` steps, and then
the sharded fp32 master weights are synchronised: pseudo-gradient = last synced shard - master shard,
optional anomaly skip (EWMA of the pseudo-gradient norm over the shard group), reduction over the
replica group (mean, or linear / GTA reducers, optionally weighted by the norm), clipping, outer
optimizer step on the last-synced shard, write-back into master and working shards. The state per rank
is only its shard. ``save_local_sgd_state_dict`` / ``load_local_sgd_state_dict`` persist
``{"global_step", "outer_optim", "local_sgd_anomaly_detector"}`` per rank.
(Reference: atorch/local_sgd/FSDP/core/_runtime_utils.py:21-188, _state_dict_utils.py:113-500.)
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from .anomaly import OnlineDynamicEWMA
from .configs import GTAConfig, LocalSGDConfig, OuterOptimizerConfig
from .reducers import build_reducer


class ShardedLocalSGD:
    def __init__(self, engine, cfg: LocalSGDConfig, outer: OuterOptimizerConfig, gta: GTAConfig):
        self.engine, self.cfg, self.outer_cfg, self.gta = engine, cfg, outer, gta
        self.replica_group = engine.cfg.replica_group
        self.replicas = engine.replicas
        self.global_step = 0
        # The baseline of the pseudo-gradient is the state at the END of the synchronous warm-up (the
        # reference creates last_synced_params lazily at its first sync, which it runs before the
        # first local step: FSDP/core/_runtime_utils.py:106). Taking it any earlier would make the
        # whole warm-up progress show up as one huge pseudo-gradient in the first outer step.
        self._symm, self._slice = None, None
        kw0 = dict(outer.outer_optim_kwargs)
        plain_sgd = outer.outer_optim_class is torch.optim.SGD and not kw0.get("weight_decay") and not kw0.get("dampening")
        if plain_sgd and self._one_kernel_possible():
            self._setup_one_kernel()
        # with the one-kernel outer step every replica keeps 1/R of the outer state of its shard
        n_state = engine.master.numel() if self._slice is None else self._slice[1] - self._slice[0]
        self.last_synced = torch.empty(n_state, dtype=torch.float32, device=engine.master.device)
        self._baseline_set = False
        if cfg.local_sgd_warmup_steps <= 0:
            self.reset_baseline()
        temp = cfg.weight_softmax_temperature
        if cfg.pseudo_gradnorm_reduce and temp is None:
            temp = 1.0
        self.reducer = build_reducer(gta, self.replica_group, temp)
        kw = dict(outer.outer_optim_kwargs)
        self.fused = None
        self.outer_optimizer = None
        self.param = torch.nn.Parameter(self.last_synced)
        if outer.outer_optim_class is torch.optim.SGD and not kw.get("weight_decay") and not kw.get("dampening"):
            self.fused = dict(lr=kw.get("lr", 1.0), momentum=kw.get("momentum", 0.0), nesterov=bool(kw.get("nesterov")))
            self.momentum = torch.zeros_like(self.last_synced)
        elif outer.outer_optim_class is not None:
            self.outer_optimizer = outer.outer_optim_class([self.param], **kw)
        self.outer_steps = 0
        self.detector = OnlineDynamicEWMA(cfg.ewma_alpha, cfg.ewma_warmup_steps, cfg.ewma_threshold) \
            if cfg.skip_anomaly else None

    def _one_kernel_possible(self) -> bool:
        """The whole outer step as ONE kernel over peer memory (csrc/comm.cu p2p_allreduce_nesterov_kernel):
        plain SGD/Nesterov, no reducer / anomaly skipping / clipping, 2..8 replicas on one NVSwitch domain."""
        cfg, eng = self.cfg, self.engine
        if not eng.on_cuda or self.replicas < 2 or self.replicas > 8 or cfg.skip_anomaly or cfg.pseudo_gradnorm_reduce \
                or cfg.clip_pseudo_grad is not None or self.gta.reducer is not None \
                or os.environ.get("ATB_FUSED_COMM", "1") == "0":
            return False
        from ..parallel import symm

        return symm.available()

    def _setup_one_kernel(self) -> None:
        from ..parallel import symm

        eng, R = self.engine, self.replicas
        n = (eng.master.numel() + 4 * R - 1) // (4 * R) * (4 * R)
        try:
            self._symm = symm.SymmetricBuffer(n, torch.float32, self.replica_group, eng.device)
        except Exception:
            self._symm = None
            return
        r = dist.get_rank(self.replica_group)
        self._slice = (r * (n // R), (r + 1) * (n // R))

    def _master_slice(self) -> torch.Tensor:
        """This rank's part of the (zero-padded) master shard, as the outer state is laid out."""
        m = self.engine.master
        if self._slice is None:
            return m
        lo, hi = self._slice
        out = torch.zeros(hi - lo, dtype=m.dtype, device=m.device)
        e = min(hi, m.numel())
        if e > lo:
            out[: e - lo] = m[lo:e]
        return out

    def skip_replica_reduce(self) -> bool:
        """Replica all-reduce of gradients is needed only during the synchronous warm-up."""
        return self.global_step >= self.cfg.local_sgd_warmup_steps

    def should_sync(self) -> bool:
        s, w = self.global_step, self.cfg.local_sgd_warmup_steps
        return s >= w and (s - w) % self.cfg.local_sgd_sync_interval == 0

    @torch.no_grad()
    def after_optimizer_step(self) -> None:
        if self.should_sync() and self.replicas > 1:
            self.sync()
        self.global_step += 1
        if not self._baseline_set and self.global_step >= self.cfg.local_sgd_warmup_steps:
            self.reset_baseline()                     # last synchronous step done: replicas are identical

    @torch.no_grad()
    def sync(self) -> None:
        eng, cfg = self.engine, self.cfg
        if not self._baseline_set:
            self.reset_baseline()
        if self._symm is not None:
            buf, f, n = self._symm, self.fused, eng.master.numel()
            buf.wait_peers_done()
            buf.tensor[:n].copy_(eng.master)
            if n < buf.numel:
                buf.tensor[n:].zero_()
            buf.allreduce_nesterov(self.last_synced, self.momentum, f["lr"], f["momentum"], f["nesterov"],
                                   self.outer_steps == 0 or f["momentum"] == 0.0)
            self.outer_steps += 1
            eng.master.copy_(buf.tensor[:n])
            eng.sync_working_copy()
            return
        pg = self.last_synced - eng.master
        kw = {}
        if cfg.skip_anomaly or cfg.pseudo_gradnorm_reduce or cfg.clip_pseudo_grad is not None:
            sq = ops.sum_squares(pg)
            if eng.world > 1:
                dist.all_reduce(sq, group=eng.group)
            norm = sq.sqrt()
            if cfg.skip_anomaly:
                if self.detector.is_outlier(norm):
                    pg.zero_()
                    norm = norm + 1e6
                else:
                    self.detector.update(norm)
            if cfg.pseudo_gradnorm_reduce:
                kw["weight"] = -norm
        if self.reducer is None:
            pg.div_(self.replicas)
            dist.all_reduce(pg, group=self.replica_group)
        else:
            self.reducer.reduce_tensor(pg, **kw)
        scale = 1.0
        if cfg.clip_pseudo_grad is not None:
            sq = ops.sum_squares(pg)
            if eng.world > 1:
                dist.all_reduce(sq, group=eng.group)
            scale = float(torch.clamp(cfg.clip_pseudo_grad / (sq.sqrt() + 1e-6), max=1.0))
        if self.fused is not None:
            f = self.fused
            ops.outer_sgd_step(self.last_synced, self.momentum, pg, None, f["lr"], f["momentum"], f["nesterov"],
                               self.outer_steps == 0 or f["momentum"] == 0.0, scale)
        elif self.outer_optimizer is not None:
            self.param.grad = pg.mul_(scale)
            self.outer_optimizer.step()
            self.param.grad = None
        else:
            self.last_synced.sub_(pg)
        self.outer_steps += 1
        eng.master.copy_(self.last_synced)
        eng.sync_working_copy()

    @torch.no_grad()
    def reset_baseline(self) -> None:
        """Take the current master shard as the last synchronised weights (end of the warm-up, or after
        the parameters were replaced by a state-dict load)."""
        self.last_synced.copy_(self._master_slice())
        self._baseline_set = True

    def state_dict(self) -> dict:
        sd = {"global_step": self.global_step, "outer_steps": self.outer_steps,
              "last_synced": (self.last_synced if self._baseline_set else self._master_slice()).detach().cpu(),
              "state_slice": self._slice}
        if self.fused is not None:
            sd["outer_optim"] = [{"momentum_buffer": self.momentum.cpu(), "rank": self.engine.rank, **self.fused}]
        elif self.outer_optimizer is not None:
            sd["outer_optim"] = [dict(self.outer_optimizer.state_dict(), rank=self.engine.rank)]
        if self.detector is not None:
            sd["local_sgd_anomaly_detector"] = [self.detector.state_dict()]
        return sd

    def load_state_dict(self, sd: dict) -> None:
        self.global_step, self.outer_steps = sd["global_step"], sd.get("outer_steps", 0)
        self.last_synced.copy_(sd["last_synced"])
        self._baseline_set = True
        if self.fused is not None and "outer_optim" in sd:
            self.momentum.copy_(sd["outer_optim"][0]["momentum_buffer"])
        elif self.outer_optimizer is not None and "outer_optim" in sd:
            self.outer_optimizer.load_state_dict({k: v for k, v in sd["outer_optim"][0].items() if k != "rank"})
        if self.detector is not None and "local_sgd_anomaly_detector" in sd:
            self.detector.load_state_dict(sd["local_sgd_anomaly_detector"][0])


def attach_local_sgd(model, local_sgd_config=None, outer_optim_config=None, gta_config=None) -> ShardedLocalSGD:
    """Enable local SGD on a sharded model; the optimizers of :mod:`atorch_b200.parallel.fsdp` call
    ``after_optimizer_step`` through the engine."""
    eng = model.engine
    lsgd = ShardedLocalSGD(eng, local_sgd_config or LocalSGDConfig(), outer_optim_config or OuterOptimizerConfig(),
                           gta_config or GTAConfig())
    eng.local_sgd = lsgd
    return lsgd


def save_local_sgd_state_dict(model, group=None, rank0_only: bool = False, full_state_dict: bool = False,
                              cpu_offload: bool = True, save_dir: str = ".", ckpt_name: str = "local_sgd") -> str:
    lsgd = model.engine.local_sgd
    os.makedirs(save_dir, exist_ok=True)
    rank = dist.get_rank() if dist.is_initialized() else 0
    path = os.path.join(save_dir, f"{ckpt_name}_{rank:02d}.pt")
    torch.save(lsgd.state_dict(), path)
    return path


def load_local_sgd_state_dict(model, group=None, rank0_only: bool = False, full_state_dict: bool = False,
                              load_dir: str = ".", ckpt_name: str = "local_sgd") -> None:
    rank = dist.get_rank() if dist.is_initialized() else 0
    model.engine.local_sgd.load_state_dict(torch.load(os.path.join(load_dir, f"{ckpt_name}_{rank:02d}.pt"),
                                                      weights_only=False))
