"""Logging helpers: the ``atorch.logger`` logger, rank-0 / once logging, timers and a TensorBoard
writer wrapper. (Reference: atorch/common/log_utils.py:12-123.)"""
from __future__ import annotations

import logging
import sys
import time
from collections import defaultdict
from typing import Dict, Optional

_FMT = "[%(asctime)s] [%(levelname)s] [%(filename)s:%(lineno)d:%(funcName)s] %(message)s"
default_logger = logging.getLogger("atorch.logger")
if not default_logger.handlers:
    _h = logging.StreamHandler(sys.stderr)
    _h.setFormatter(logging.Formatter(_FMT))
    default_logger.addHandler(_h)
    default_logger.setLevel(logging.INFO)
    default_logger.propagate = False

_once = set()


def log_rank_0(msg: str, level: int = logging.INFO) -> None:
    from ..distributed.distributed import rank

    if rank() in (None, 0):
        default_logger.log(level, msg)


def log_once(msg: str, level: int = logging.INFO) -> None:
    if msg not in _once:
        _once.add(msg)
        default_logger.log(level, msg)


class Timer:
    def __init__(self, name: str, stats: Optional["TimeStats"] = None):
        self.name, self.stats = name, stats
        self.elapsed = 0.0

    def __enter__(self):
        self._t0 = time.time()
        return self

    def __exit__(self, *exc):
        self.elapsed = time.time() - self._t0
        if self.stats is not None:
            self.stats.add(self.name, self.elapsed)
        return False


class TimeStats:
    def __init__(self, name: str = ""):
        self.name = name
        self.records: Dict[str, list] = defaultdict(list)

    def add(self, key: str, value: float) -> None:
        self.records[key].append(value)

    def mean(self, key: str) -> float:
        v = self.records.get(key, [])
        return sum(v) / len(v) if v else 0.0

    def summary(self) -> Dict[str, float]:
        return {k: self.mean(k) for k in self.records}


class DashBoardWriter:
    """TensorBoard scalar writer that degrades to a no-op when tensorboard is not installed."""

    def __init__(self, logdir: str = "./"):
        try:
            from torch.utils.tensorboard import SummaryWriter

            self.writer = SummaryWriter(logdir)
        except Exception:
            self.writer = None

    def add_scalars(self, stats: Dict[str, float], n_iter: int) -> None:
        if self.writer is not None:
            for k, v in stats.items():
                self.writer.add_scalar(k, v, n_iter)

    def flush(self) -> None:
        if self.writer is not None:
            self.writer.flush()
