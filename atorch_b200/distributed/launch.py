"""Static multi-process launcher with failure monitoring and relaunch on hang.

``launch(nproc_per_node, script, args, ...)`` starts one process per local rank with the usual
environment (RANK, LOCAL_RANK, WORLD_SIZE, MASTER_ADDR/PORT, NPROC_PER_NODE, NODE_SIZE), watches
them, kills the rest when one fails and restarts the whole group up to ``max_restarts`` times. With
``relaunch_on_hanging`` it also hosts the key-value store of the hanging detectors and restarts the
workers when one of them reports a hang.
(Reference: atorch/distributed/launch.py:178-361 static launcher; atorch/fault_tolerance/
custom_agent.py:92-139 relaunch loop.)
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import time
from typing import Dict, List, Optional

from .distributed import find_free_port


class WorkerGroup:
    def __init__(self, cmd: List[str], nproc: int, node_rank: int, nnodes: int, master_addr: str, master_port: int,
                 extra_env: Optional[Dict[str, str]] = None, rank_log_dir: Optional[str] = None):
        self.cmd, self.nproc, self.node_rank, self.nnodes = cmd, nproc, node_rank, nnodes
        self.master_addr, self.master_port = master_addr, master_port
        self.extra_env, self.rank_log_dir = extra_env or {}, rank_log_dir
        self.procs: List[subprocess.Popen] = []
        self._logs = []

    def start(self) -> None:
        world = self.nproc * self.nnodes
        for lr in range(self.nproc):
            env = dict(os.environ)
            env.update(RANK=str(self.node_rank * self.nproc + lr), LOCAL_RANK=str(lr), WORLD_SIZE=str(world),
                       MASTER_ADDR=self.master_addr, MASTER_PORT=str(self.master_port),
                       NPROC_PER_NODE=str(self.nproc), LOCAL_WORLD_SIZE=str(self.nproc), NODE_SIZE=str(self.nnodes),
                       NODE_RANK=str(self.node_rank))
            env.update(self.extra_env)
            out = None
            if self.rank_log_dir:
                os.makedirs(self.rank_log_dir, exist_ok=True)
                out = open(os.path.join(self.rank_log_dir, f"rank_{env['RANK']}.log"), "ab")
                self._logs.append(out)
            self.procs.append(subprocess.Popen(self.cmd, env=env, stdout=out, stderr=subprocess.STDOUT if out else None,
                                               start_new_session=True))

    def poll(self):
        """None while all run; 0 when all exited cleanly; otherwise the first non-zero exit code."""
        codes = [p.poll() for p in self.procs]
        bad = [c for c in codes if c not in (None, 0)]
        if bad:
            return bad[0]
        return 0 if all(c == 0 for c in codes) else None

    def kill(self) -> None:
        for p in self.procs:            # only the exact processes started here
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        deadline = time.time() + 10
        for p in self.procs:
            try:
                p.wait(timeout=max(0.1, deadline - time.time()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
        for f in self._logs:
            f.close()
        self.procs, self._logs = [], []


def launch(cmd: List[str], nproc_per_node: int = 1, nnodes: int = 1, node_rank: int = 0,
           master_addr: str = "127.0.0.1", master_port: Optional[int] = None, max_restarts: int = 0,
           monitor_interval: float = 1.0, relaunch_on_hanging: bool = False, rank_log_dir: Optional[str] = None) -> int:
    master_port = master_port or find_free_port()
    extra, status, store = {}, None, None
    if relaunch_on_hanging:
        import datetime

        from torch.distributed import TCPStore

        from ..fault_tolerance.hanging_detector import RelaunchStatus

        sport = find_free_port()
        store = TCPStore("127.0.0.1", sport, is_master=True, timeout=datetime.timedelta(seconds=30),
                         wait_for_workers=False)
        extra.update(TORCHELASTIC_AGENT_MASTER_ADDR="127.0.0.1", TORCHELASTIC_AGENT_MASTER_PORT=str(sport),
                     NCCL_ASYNC_ERROR_HANDLING="1")
        status = RelaunchStatus("agent", world_size=nproc_per_node * nnodes, store=store)
    restarts = 0
    while True:
        group = WorkerGroup(cmd, nproc_per_node, node_rank, nnodes, master_addr, master_port, extra, rank_log_dir)
        group.start()
        code, hang = None, False
        while code is None:
            time.sleep(monitor_interval)
            code = group.poll()
            if status is not None and status.should_relaunch():
                hang = True
                break
        group.kill()
        if code == 0 and not hang:
            return 0
        if restarts >= max_restarts:
            return code if code not in (None, 0) else 1
        restarts += 1
        if status is not None:
            status.step_relaunch()
        master_port = find_free_port()
