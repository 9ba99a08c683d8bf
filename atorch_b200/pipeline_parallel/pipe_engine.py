"""``PipeEngine``: a pipe module plus a scheduler configuration behind one call, ``train_batch_step(data_iter)``.

The configuration (a dict, or the path of a yaml / json file) names the scheduler (``ForwardBackwardNoPipelinging``,
``OneForwardOneBackward``, ``OneForwardOneBackwardInterleaving``), ``global_batchsize`` and ``micro_batchsize`` (their
ratio over the data-parallel size is the number of micro-batches), ``virtual_pp_size``, ``device`` and
``return_average_loss``. ``train_batch_step`` pulls the micro-batches of one step from the iterator (for the
interleaved scheduler a list of ``virtual_pp_size`` iterators is accepted; the first feeds the inputs), runs forward and
backward of all of them through the schedule and returns the per-micro-batch losses on the last stage (their mean with
``return_average_loss``), ``[]`` elsewhere.
(Reference: atorch/pipeline_parallel/pipe_engine.py:17-89, scheduler.py:15-25; the reference's 1F1B executors are
empty stubs, the schedules here are the ones of ``pipe_schedule.py``.)
"""
from __future__ import annotations

import logging
from enum import Enum
from typing import Iterable, List, Union

import torch

from ..distributed import distributed as D
from ..utils.config import Config
from .pipe_schedule import PipelineSchedule

logger = logging.getLogger("atorch.logger")


class P2PType(Enum):
    SEND = "send"
    RECV = "recv"


class PipeSchedulerType(Enum):
    ForwardBackwardNoPipelinging = "ForwardBackwardNoPipelinging"
    OneForwardOneBackward = "OneForwardOneBackward"
    OneForwardOneBackwardInterleaving = "OneForwardOneBackwardInterleaving"


_KIND = {PipeSchedulerType.ForwardBackwardNoPipelinging: "ScheduleGPipe",
         PipeSchedulerType.OneForwardOneBackward: "Schedule1F1B",
         PipeSchedulerType.OneForwardOneBackwardInterleaving: "ScheduleInterleaved1F1B"}


def is_batch_on_device(batch, device) -> bool:
    """True when every tensor of a (nested) batch already lives on ``device``."""
    device = torch.device(device)
    if isinstance(batch, torch.Tensor):
        return batch.device.type == device.type and (device.index is None or batch.device.index == device.index)
    if isinstance(batch, dict):
        return all(is_batch_on_device(v, device) for v in batch.values())
    if isinstance(batch, (list, tuple)):
        return all(is_batch_on_device(v, device) for v in batch)
    return True


def _to_device(batch, device):
    if isinstance(batch, torch.Tensor):
        return batch.to(device, non_blocking=True)
    if isinstance(batch, dict):
        return {k: _to_device(v, device) for k, v in batch.items()}
    if isinstance(batch, (list, tuple)):
        return type(batch)(_to_device(v, device) for v in batch)
    return batch


class PipeEngine:
    def __init__(self, pipe_module, config: Union[str, dict]):
        self.config = self._parse_config(config)
        self.model = pipe_module.to(self.config.device)
        dp = D.parallel_group_size("data") or 1
        self.n_microbatches = max(1, self.config.global_batchsize // (self.config.micro_batchsize * dp))
        kind = _KIND[self.config.scheduler]
        if kind == "Schedule1F1B" and len(pipe_module.stages) > 1:
            kind = "ScheduleInterleaved1F1B"
        loss_fn = pipe_module.loss_func if pipe_module.loss_func is not None else pipe_module.ori_loss_func
        self.schedule = PipelineSchedule(pipe_module.stages, self.n_microbatches, loss_fn, kind, pipe_module.pp_rank,
                                         pipe_module.pp_size)

    @classmethod
    def _parse_config(cls, input_config: Union[str, dict]) -> Config:
        if isinstance(input_config, str):
            config = Config.from_file(input_config)
        elif isinstance(input_config, dict):
            config = Config(input_config)
        else:
            raise ValueError("Config must be a string or a dictionary")
        if "scheduler" in config:
            config.scheduler = PipeSchedulerType(getattr(config.scheduler, "value", config.scheduler))
        else:
            logger.warning("Missing scheduler in PipeEngine config, set it to ForwardBackwardNoPipelinging.")
            config.scheduler = PipeSchedulerType.ForwardBackwardNoPipelinging
        for key, default in (("return_average_loss", False), ("virtual_pp_size", 1),
                             ("device", "cuda" if torch.cuda.is_available() else "cpu")):
            if key not in config:
                setattr(config, key, default)
        for key, default in (("global_batchsize", 8), ("micro_batchsize", 1)):
            if key not in config:
                logger.warning("Missing %s in PipeEngine config, set it to %d.", key, default)
                setattr(config, key, default)
        return config

    def _micro_batches(self, data_iter) -> List:
        it = iter(data_iter)
        return [_to_device(next(it), self.config.device) for _ in range(self.n_microbatches)]

    def train_batch_step(self, data_iter: Union[Iterable, List[Iterable]]):
        if self.config.scheduler is PipeSchedulerType.OneForwardOneBackwardInterleaving and isinstance(data_iter, list):
            assert len(data_iter) == self.config.virtual_pp_size
            data_iter = data_iter[0]
        mbs = self._micro_batches(data_iter)
        first = mbs[0]
        if isinstance(first, dict):
            target = torch.cat([m.pop("labels") for m in mbs]) if "labels" in first else None
            kwargs = {k: torch.cat([m[k] for m in mbs]) for k in first if k != "labels"}
            args = ()
        else:
            cols = list(zip(*[m if isinstance(m, (list, tuple)) else (m,) for m in mbs]))
            target = torch.cat(cols[-1]) if len(cols) > 1 else None
            args = tuple(torch.cat(c) for c in (cols[:-1] if len(cols) > 1 else cols))
            kwargs = {}
        losses: List[torch.Tensor] = []
        self.schedule.step(*args, target=target, losses=losses, **kwargs)
        if self.config.return_average_loss and losses:
            return torch.stack(losses).mean()
        return losses
