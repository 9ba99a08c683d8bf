"""Network traffic monitor: a thread samples the byte counters of InfiniBand / NVLink-adjacent NICs under
``/sys/class/infiniband/*/ports/*/counters`` and writes chrome-trace counter events (``--ib_stat_kw
interval,count,path`` of the launcher). (Reference: atorch/utils/ib_monitor.py:12-178.)"""
from __future__ import annotations

import glob
import json
import threading
import time
from typing import Dict, List, Optional


def read_counters(root: str = "/sys/class/infiniband") -> Dict[str, int]:
    out = {}
    for f in glob.glob(f"{root}/*/ports/*/counters/port_*_data"):
        try:
            with open(f) as fh:
                out[f[len(root) + 1:]] = int(fh.read().strip()) * 4       # counters are in 4-byte words
        except (OSError, ValueError):
            pass
    return out


class IBMonitor:
    def __init__(self, interval: float = 1.0, count: int = 0, path: Optional[str] = None, root: str = "/sys/class/infiniband"):
        self.interval, self.count, self.path, self.root = interval, count, path, root
        self.events: List[dict] = []
        self._stop = threading.Event()
        self.thread: Optional[threading.Thread] = None

    def _run(self):
        prev, n = read_counters(self.root), 0
        while not self._stop.wait(self.interval):
            cur = read_counters(self.root)
            ts = time.time() * 1e6
            for k, v in cur.items():
                self.events.append({"name": k, "ph": "C", "ts": ts, "pid": 0,
                                    "args": {"bytes_per_s": (v - prev.get(k, v)) / self.interval}})
            prev, n = cur, n + 1
            if self.count and n >= self.count:
                break
        if self.path:
            with open(self.path, "w") as f:
                json.dump({"traceEvents": self.events}, f)

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(self.interval * 2 + 1)
