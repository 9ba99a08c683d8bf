"""Tasks the acceleration engine hands to worker processes.
(Reference: atorch/auto/engine/task.py:1-63.)"""
from __future__ import annotations

from typing import Any, List, Optional


class TaskType:
    ANALYSE = "ANALYSE"
    TUNE = "TUNE"
    FINISH = "FINISH"
    SETUP_PARALLEL_GROUP = "SETUP_PARALLEL_GROUP"
    DRYRUN = "DRYRUN"
    WAIT = "WAIT"
    FAIL = "FAIL"


class TaskProcessMode:
    ONE_PROCESS = "ONE_PROCESS"     # any single idle process runs it
    ALL_PROCESS = "ALL_PROCESS"     # every process runs it, starting only when all are idle


class TaskStatus:
    PENDING, ASSIGNING, RUNNING, CANCELLED, FAILED, SUCCEEDED = range(6)


class Task:
    """ONE_PROCESS: PENDING -> RUNNING -> SUCCEEDED | FAILED;
    ALL_PROCESS: PENDING -> ASSIGNING (handed out process by process) -> RUNNING -> SUCCEEDED | FAILED."""

    def __init__(self, task_type: str, task_info: Any = None, task_id: int = -1, strategy_id: int = -1,
                 process_mode: str = TaskProcessMode.ONE_PROCESS, time_limit: Optional[float] = None):
        self.task_id, self.task_type, self.task_info = task_id, task_type, task_info
        self.strategy_id, self.process_mode, self.time_limit = strategy_id, process_mode, time_limit
        self.process_assigned: List[int] = []
        self.reported: List[int] = []
        self.status = TaskStatus.PENDING
        self.task_result: Any = None

    def __repr__(self) -> str:
        return f"Task({self.task_id}, {self.task_type}, strategy={self.strategy_id}, mode={self.process_mode})"
