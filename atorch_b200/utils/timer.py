"""Throughput / step timers. ``ThroughputTimer`` counts samples per second over log intervals
(reference: atorch/utils/timer.py:8-77); ``DeviceStepTimer`` times steps on the device with CUDA
events and reduces with MAX over ranks, which is how every multi-GPU number of this framework is taken.
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch
import torch.distributed as dist


class ThroughputTimer:
    def __init__(self, batch_size: int, start_step: int = 2, steps_per_output: int = 50, monitor_memory: bool = False,
                 logging_fn=None):
        self.batch_size, self.start_step, self.steps_per_output = max(batch_size, 1), start_step, steps_per_output
        self.monitor_memory, self.logging = monitor_memory, logging_fn or print
        self.global_step_count = self.micro_step_count = 0
        self.total_elapsed_time = self.step_elapsed_time = 0.0
        self.started, self.start_time = False, 0.0

    def _sync(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def start(self):
        self.started = True
        if self.global_step_count >= self.start_step:
            self._sync()
            self.start_time = time.time()

    def stop(self, global_step: bool = True, report_speed: bool = True):
        if not self.started:
            return
        self.started = False
        self.micro_step_count += 1
        if global_step:
            self.global_step_count += 1
        if self.start_time > 0:
            self._sync()
            d = time.time() - self.start_time
            self.total_elapsed_time += d
            self.step_elapsed_time += d
            if global_step and report_speed and self.global_step_count % self.steps_per_output == 0:
                msg = (f"step={self.global_step_count}, samples/sec={self.avg_samples_per_sec():.3f}, "
                       f"recent={self.batch_size * self.steps_per_output / max(self.step_elapsed_time, 1e-9):.3f}")
                if self.monitor_memory and torch.cuda.is_available():
                    msg += f", max_allocated_MB={torch.cuda.max_memory_allocated() / 2 ** 20:.1f}"
                self.logging(msg)
                self.step_elapsed_time = 0.0

    def avg_samples_per_sec(self) -> float:
        n = self.global_step_count - self.start_step
        if n > 0 and self.total_elapsed_time > 0:
            return self.batch_size / (self.total_elapsed_time / n)
        return float("-inf")


class DeviceStepTimer:
    """CUDA-event timing of a block of steps: ``with timer: ...`` then ``timer.ms_max_over_ranks()``."""

    def __init__(self, device=None, group=None):
        self.device, self.group = device, group
        self.ms: Optional[float] = None

    def __enter__(self):
        if dist.is_initialized():
            dist.barrier(group=self.group)
        torch.cuda.synchronize(self.device)
        self._s, self._e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._s.record()
        return self

    def __exit__(self, *exc):
        self._e.record()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        torch.cuda.synchronize(self.device)
        self.ms = self._s.elapsed_time(self._e)
        return False

    def ms_max_over_ranks(self) -> float:
        t = torch.tensor([self.ms], device=self.device or "cuda")
        if dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())
