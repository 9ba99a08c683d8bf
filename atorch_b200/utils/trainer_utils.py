"""Scheduler names of the trainer beyond the Hugging Face ones, and the messages of the asynchronous checkpoint
manager process. (Reference: atorch/utils/trainer_utils.py:9-60.)"""
from __future__ import annotations

import math
from enum import Enum
from typing import Optional

from torch.optim.lr_scheduler import LambdaLR


class AtorchSchedulerType(str, Enum):
    LOG_WARMUP_LINEAR_DECAY = "log_warmup_linear_decay"


def log_warmup_linear_decay_factor(step: int, num_warmup_steps: int, num_training_steps: int) -> float:
    """0 at step 0, ``log(step) / log(warmup)`` during warm-up (so 0 again at step 1, 1 at the end of warm-up), then
    a straight line to 0 at ``num_training_steps``."""
    if step == 0:
        return 0.0
    if step < num_warmup_steps:
        return math.log(step + 1e-6) / math.log(num_warmup_steps + 1e-6)
    return max(0.0, float(num_training_steps - step) / float(max(1, num_training_steps - num_warmup_steps)))


def get_linear_schedule_with_log_warmup(optimizer, num_warmup_steps, num_training_steps, last_epoch=-1):
    return LambdaLR(optimizer, lambda s: log_warmup_linear_decay_factor(s, num_warmup_steps, num_training_steps),
                    last_epoch)


TYPE_TO_ATORCHSCHEDULER_FUNCTION = {AtorchSchedulerType.LOG_WARMUP_LINEAR_DECAY: get_linear_schedule_with_log_warmup}
ATORCHSCHEDULER_NAMES = [t.value for t in AtorchSchedulerType]


def _hf_scheduler_names():
    try:
        from transformers.trainer_utils import SchedulerType

        return [t.value for t in SchedulerType]
    except ImportError:
        return []


SCHEDULER_NAMES = _hf_scheduler_names()


def get_scheduler(name, optimizer, num_warmup_steps, num_training_steps):
    """A Hugging Face schedule by name, or one of this package's."""
    name = getattr(name, "value", name)
    if name in ATORCHSCHEDULER_NAMES:
        return TYPE_TO_ATORCHSCHEDULER_FUNCTION[AtorchSchedulerType(name)](optimizer, num_warmup_steps,
                                                                           num_training_steps)
    if name in SCHEDULER_NAMES:
        from transformers import get_scheduler as hf_get_scheduler

        return hf_get_scheduler(name, optimizer, num_warmup_steps, num_training_steps)
    raise ValueError(f"{name} is not a valid schedule name, please select one of "
                     f"{SCHEDULER_NAMES + ATORCHSCHEDULER_NAMES}.")


class AsyncCheckpointSignal(Enum):
    DELETE_CKPT = 1      # the manager process deletes a checkpoint
    SAVE_OVER = 2        # a saving process has finished: reap it
    TRAIN_OVER = 3       # training ends: the manager exits


class PipeMessageEntity:
    def __init__(self, signal_type: AsyncCheckpointSignal, pid: Optional[int] = None, ckpt_path: Optional[str] = None):
        self.signal_type, self.pid, self.ckpt_path = signal_type, pid, ckpt_path
