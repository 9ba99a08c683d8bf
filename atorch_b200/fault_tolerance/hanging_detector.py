"""Hang detection and coordinated relaunch.

Workers run a ``HangingDetector``: a daemon thread that expects ``report_normal()`` at least every
``timeout`` seconds while running. When the reports stop, the worker raises its *relaunch id* in a
key-value store shared with the launcher agent (``RelaunchStatus``); the agent polls
``should_relaunch()`` (some worker id above its own) and restarts all workers. Everything lives on
the host: the store is a ``torch.distributed.TCPStore`` (address from
``TORCHELASTIC_AGENT_MASTER_ADDR/PORT``) or any object with ``set/get``.
(Reference: atorch/fault_tolerance/hanging_detector.py:16-145, custom_agent.py:25-201.)
"""
from __future__ import annotations

import datetime
import os
import threading
import time
from typing import Optional


class RelaunchStatus:
    PREFIX = "relaunch_status/"

    def __init__(self, role: str, worker_rank: Optional[int] = None, world_size: Optional[int] = None, store=None):
        assert role in ("worker", "agent")
        self.role, self.worker_rank = role, worker_rank
        self.world_size = world_size if world_size is not None else int(os.environ.get("WORLD_SIZE", "1"))
        self.relaunch_id = 0
        self.store = store if store is not None else self._store_from_env()
        self.initialized = self.store is not None
        if self.initialized and role == "worker":
            self.relaunch_id = self._get(f"agent", 0)
            self._set(f"worker_{worker_rank}", self.relaunch_id)

    @staticmethod
    def _store_from_env():
        addr, port = os.environ.get("TORCHELASTIC_AGENT_MASTER_ADDR"), os.environ.get("TORCHELASTIC_AGENT_MASTER_PORT")
        if not addr or not port:
            return None
        from torch.distributed import TCPStore

        return TCPStore(addr, int(port), is_master=False, timeout=datetime.timedelta(seconds=30))

    def _set(self, key: str, value: int) -> None:
        self.store.set(self.PREFIX + key, str(value))

    def _get(self, key: str, default: int) -> int:
        try:
            if hasattr(self.store, "check") and not self.store.check([self.PREFIX + key]):
                return default
            v = self.store.get(self.PREFIX + key)
            return int(v.decode() if isinstance(v, bytes) else v)
        except Exception:
            return default

    def set_relaunch(self) -> None:
        """Worker side: ask for a relaunch."""
        self.relaunch_id += 1
        self._set(f"worker_{self.worker_rank}", self.relaunch_id)

    def should_relaunch(self) -> bool:
        """Agent side: has any worker asked for a relaunch newer than the last one performed?"""
        ids = [self._get(f"worker_{r}", 0) for r in range(self.world_size)]
        return max(ids) > self.relaunch_id

    def step_relaunch(self) -> None:
        """Agent side: a relaunch was performed."""
        self.relaunch_id += 1
        self._set("agent", self.relaunch_id)


class HangingDetector:
    def __init__(self, timeout: float = 300, monitor_interval: float = 15, rank: Optional[int] = None, store=None,
                 on_hang=None):
        self.timeout, self.monitor_interval = timeout, monitor_interval
        self.worker_rank = rank if rank is not None else int(os.environ.get("RANK", "0"))
        self.relaunch_status = RelaunchStatus("worker", worker_rank=self.worker_rank, store=store)
        if not self.relaunch_status.initialized:
            raise RuntimeError("Initialize HangingDetector failed. Launch the training script with "
                               "'python -m atorch.distributed.run --relaunch_on_hanging train_script.py'")
        self.on_hang = on_hang
        self._last_report_time = None
        self.is_running = False
        self.enabled = None
        self.thread: Optional[threading.Thread] = None
        self.hang_detected = False

    def start(self) -> None:
        if self.enabled is None:
            self.enabled = True
        if not self.is_running:
            self._last_report_time = time.time()
            self.is_running = True
            if self.enabled and self.thread is None:
                self.thread = threading.Thread(target=self._watch, daemon=True)
                self.thread.start()

    def stop(self, finalize: bool = False) -> None:
        self.is_running = False
        if finalize:
            self.enabled = False

    def report_normal(self) -> None:
        self._last_report_time = time.time()

    def _watch(self) -> None:
        while self.enabled:
            time.sleep(self.monitor_interval)
            if self.is_running and time.time() - self._last_report_time > self.timeout:
                self.hang_detected = True
                self.relaunch_status.set_relaunch()
                if self.on_hang is not None:
                    self.on_hang()
                break
