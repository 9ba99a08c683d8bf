"""``python -m atorch_b200.distributed.run [options] script.py [script args]``.

Modes: the default static launcher (one process per local rank, kill-all on first failure,
``--max_restarts``), ``--fault_tolerant`` / ``--elastic`` (restart the worker group on failure, up to
100 times by default) and ``--relaunch_on_hanging`` (workers run a ``HangingDetector``; a reported
hang restarts the group). ``--rank_log_dir`` redirects each rank's output to its own file.
(Reference: atorch/distributed/run.py:347-404.)
"""
from __future__ import annotations

import argparse
import sys
from argparse import REMAINDER

from .launch import launch


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="atorch_b200 launcher")
    p.add_argument("--nnodes", type=int, default=1)
    p.add_argument("--nproc_per_node", "--nproc-per-node", type=int, default=1)
    p.add_argument("--node_rank", "--node-rank", type=int, default=0)
    p.add_argument("--master_addr", "--master-addr", type=str, default="127.0.0.1")
    p.add_argument("--master_port", "--master-port", type=int, default=None)
    p.add_argument("--max_restarts", "--max-restarts", type=int, default=None)
    p.add_argument("--monitor_interval", "--monitor-interval", type=float, default=1.0)
    p.add_argument("--elastic", action="store_true")
    p.add_argument("--fault_tolerant", action="store_true")
    p.add_argument("--relaunch_on_hanging", action="store_true")
    p.add_argument("--rank_log_dir", type=str, default=None)
    p.add_argument("-m", "--module", action="store_true", help="treat the script as a python module")
    p.add_argument("--no_python", action="store_true")
    p.add_argument("training_script", type=str)
    p.add_argument("training_script_args", nargs=REMAINDER)
    return p.parse_args(argv)


def main(argv=None) -> int:
    a = parse_args(argv)
    if a.no_python:
        cmd = [a.training_script]
    elif a.module:
        cmd = [sys.executable, "-u", "-m", a.training_script]
    else:
        cmd = [sys.executable, "-u", a.training_script]
    cmd += a.training_script_args
    restarts = a.max_restarts if a.max_restarts is not None else (100 if (a.elastic or a.fault_tolerant) else
                                                                 (3 if a.relaunch_on_hanging else 0))
    return launch(cmd, a.nproc_per_node, a.nnodes, a.node_rank, a.master_addr, a.master_port, restarts,
                  a.monitor_interval, a.relaunch_on_hanging, a.rank_log_dir)


if __name__ == "__main__":
    sys.exit(main())
