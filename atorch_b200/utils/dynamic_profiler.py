"""On-demand profiling of a running job, driven by a JSON config file.

A monitor thread polls ``config_path`` (``ThreadFileConfigMonitor``); when its content changes, a
profiling *session* is scheduled: ``{"start_step": N, "steps": K, "ranks": [..] | "all", "output_dir": ...,
"with_stack": bool}``. ``DynamicProfiler.step()`` (call once per optimizer step, or let
``patch_step_function(optimizer)`` do it) starts a ``torch.profiler`` window at ``start_step`` on the chosen
ranks and exports a chrome trace after ``steps`` steps. Per-rank session state is written next to the
config (``.dynamic_profile_state.<rank>.json``) so an external tool can see progress.
(Reference: atorch/utils/dynamic_profiler/_dynamic_profile.py:105-650, _file_monitor.py:74-222.)"""
from __future__ import annotations

import json
import os
import threading
import time
from typing import Callable, Optional

import torch


class ThreadFileConfigMonitor:
    def __init__(self, path: str, on_change: Callable[[dict], None], poll_interval: float = 1.0):
        self.path, self.on_change, self.poll_interval = path, on_change, poll_interval
        self._mtime = None
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)

    def start(self):
        self.thread.start()

    def stop(self):
        self._stop.set()

    def poll_once(self) -> bool:
        try:
            m = os.stat(self.path).st_mtime_ns
        except OSError:
            return False
        if m == self._mtime:
            return False
        self._mtime = m
        try:
            with open(self.path) as f:
                self.on_change(json.load(f))
            return True
        except (OSError, ValueError):
            return False

    def _run(self):
        while not self._stop.wait(self.poll_interval):
            self.poll_once()


class DynamicProfiler:
    IDLE, SCHEDULED, RUNNING, DONE = "idle", "scheduled", "running", "done"

    def __init__(self, config_path: str, rank: int = 0, poll_interval: float = 1.0, start_monitor: bool = True):
        self.config_path, self.rank = config_path, rank
        self.step_count, self.state, self.session, self.profiler = 0, self.IDLE, None, None
        self.lock = threading.Lock()
        self.monitor = ThreadFileConfigMonitor(config_path, self._on_config, poll_interval)
        if start_monitor:
            self.monitor.start()

    def _on_config(self, cfg: dict) -> None:
        ranks = cfg.get("ranks", "all")
        if ranks != "all" and self.rank not in ranks:
            return
        with self.lock:
            if self.state in (self.RUNNING,):
                return
            self.session = {"start_step": int(cfg.get("start_step", self.step_count + 1)),
                            "steps": int(cfg.get("steps", 1)),
                            "output_dir": cfg.get("output_dir", os.path.dirname(self.config_path) or "."),
                            "with_stack": bool(cfg.get("with_stack", False))}
            self.state = self.SCHEDULED
            self._write_state()

    def _write_state(self) -> None:
        f = os.path.join(os.path.dirname(self.config_path) or ".", f".dynamic_profile_state.{self.rank}.json")
        try:
            with open(f, "w") as fh:
                json.dump({"state": self.state, "step": self.step_count, "session": self.session}, fh)
        except OSError:
            pass

    def step(self) -> None:
        with self.lock:
            self.step_count += 1
            s = self.session
            if self.state == self.SCHEDULED and self.step_count >= s["start_step"]:
                acts = [torch.profiler.ProfilerActivity.CPU]
                if torch.cuda.is_available():
                    acts.append(torch.profiler.ProfilerActivity.CUDA)
                self.profiler = torch.profiler.profile(activities=acts, with_stack=s["with_stack"])
                self.profiler.start()
                self.state, s["end_step"] = self.RUNNING, self.step_count + s["steps"]
                self._write_state()
            elif self.state == self.RUNNING and self.step_count >= s["end_step"]:
                self.profiler.stop()
                os.makedirs(s["output_dir"], exist_ok=True)
                out = os.path.join(s["output_dir"], f"trace_rank{self.rank}_step{self.step_count}.json")
                self.profiler.export_chrome_trace(out)
                s["trace"] = out
                self.profiler, self.state = None, self.DONE
                self._write_state()

    def patch_step_function(self, optimizer) -> None:
        orig = optimizer.step

        def step(*a, **k):
            r = orig(*a, **k)
            self.step()
            return r
        optimizer.step = step

    def close(self) -> None:
        self.monitor.stop()


_GLOBAL: Optional[DynamicProfiler] = None


def init(config_path: str, rank: Optional[int] = None, poll_interval: float = 1.0) -> DynamicProfiler:
    """Process-wide dynamic profiler (the form the trainer's profiler callback uses); ``step()`` below
    advances it. (Reference: atorch/utils/dynamic_profiler/__init__.py ``init`` / ``step``.)"""
    global _GLOBAL
    if _GLOBAL is not None:
        _GLOBAL.close()
    if rank is None:
        rank = int(os.environ.get("RANK", "0"))
    _GLOBAL = DynamicProfiler(config_path, rank=rank, poll_interval=poll_interval)
    return _GLOBAL


def step() -> None:
    if _GLOBAL is not None:
        _GLOBAL.step()
