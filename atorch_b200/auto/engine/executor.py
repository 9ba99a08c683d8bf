"""Task queue of the acceleration engine: the state machine behind ``get_task`` / ``report_task_result``.

The search is a coroutine-like plan: ANALYSE (one process) → for each candidate strategy, SETUP_PARALLEL_GROUP
(all processes; dropped when the parallel mode is the one already set up) then TUNE (only for candidates
with tunable methods) and DRYRUN (all processes) → FINISH with the best strategy, or FAIL. Candidates come
from the combination generator first and, when asked for, from the Bayesian generator, which proposes one
candidate at a time from the throughputs seen so far. A process that asks while nothing can be handed to it
gets a WAIT task. An ALL_PROCESS task starts only when every process is idle and is then handed to each
process once; its result is the one process 0 reports. The search ends early when ``time_limit`` expires.
(Reference: atorch/auto/engine/executor.py:36-278, planner.py:13-120, strategy.py:49-171.)
"""
from __future__ import annotations

import threading
import time
from collections import deque
from typing import Deque, Dict, List, Optional

from ..strategy import Strategy
from .task import Task, TaskProcessMode, TaskStatus, TaskType


class StrategyRecord:
    INIT, TUNED, SUCCEED, FAILED = "init", "tuned", "succeed", "failed"

    def __init__(self, strategy: Strategy, combo=None):
        self.strategy, self.combo = strategy, combo
        self.status = self.TUNED if not any(t for _, _, t in strategy) else self.INIT
        self.dryrun_result: Optional[dict] = None

    @property
    def throughput(self) -> float:
        return float((self.dryrun_result or {}).get("throughput", 0.0))


class Executor:
    def __init__(self, device_context: Optional[dict] = None, included_opts=None, excluded_opts=None,
                 time_limit: Optional[float] = None, load_strategy: Optional[Strategy] = None,
                 algo: str = "combination", verbose: bool = False):
        ctx = device_context or {"node_num": 1, "nproc_per_node": 1}
        self.total_process = int(ctx.get("node_num", 1)) * int(ctx.get("nproc_per_node", 1))
        self.device_context = ctx
        self.included, self.excluded = list(included_opts or []), list(excluded_opts or [])
        self.time_limit, self.algo, self.verbose = time_limit, algo, verbose
        self.start_time = time.time()
        self.lock = threading.Lock()
        self.tasks: Dict[int, Task] = {}
        self.pending: Deque[int] = deque()
        self.assigning: Optional[int] = None
        self.busy: Dict[int, Optional[int]] = {p: None for p in range(self.total_process)}
        self.strategies: List[StrategyRecord] = []
        self.analysis: dict = {}
        self.current_parallel_mode = None
        self.terminate_task_id: Optional[int] = None
        self._candidates: Optional[Deque[StrategyRecord]] = None
        self._sg_algo = None
        if load_strategy is not None:          # nothing to search: hand the given strategy to every process
            self.strategies.append(StrategyRecord(load_strategy))
            self.strategies[0].status = StrategyRecord.SUCCEED
            self.strategies[0].dryrun_result = {"throughput": 1.0}
            self._finish()
        else:
            self._add(Task(TaskType.ANALYSE, ["analyse_model"]))

    # ------------------------------------------------------------------ queue plumbing
    def _add(self, task: Task) -> Task:
        task.task_id = len(self.tasks)
        self.tasks[task.task_id] = task
        self.pending.append(task.task_id)
        if task.task_type in (TaskType.FINISH, TaskType.FAIL):
            self.terminate_task_id = task.task_id
        return task

    @property
    def can_be_terminated(self) -> bool:
        t = self.terminate_task_id
        return t is not None and len(self.tasks[t].process_assigned) == self.total_process

    def _expired(self) -> bool:
        return self.time_limit is not None and time.time() - self.start_time > self.time_limit

    # ------------------------------------------------------------------ planning
    def _generate_candidates(self) -> None:
        """Pick the strategy-generation algorithm; it fills ``_candidates`` stage by stage."""
        from .sg_algo import StrategyGenerationAlgorithmLibrary

        name = {"combination": "combination_sg", "bo": "bo_sg"}.get(self.algo, self.algo)
        self._sg_algo = StrategyGenerationAlgorithmLibrary()[name]
        if self._sg_algo is None:
            raise ValueError(f"unknown strategy generation algorithm {self.algo!r}")
        self._candidates = deque()

    def _next_candidate(self) -> Optional[StrategyRecord]:
        if self._expired():
            return None
        if not self._candidates and not self._sg_algo.is_done:
            self._sg_algo(self)
        return self._candidates.popleft() if self._candidates else None

    def _schedule_strategy(self, rec: StrategyRecord) -> None:
        sid = len(self.strategies)
        self.strategies.append(rec)
        found, mode = rec.strategy.get_parallel_mode()
        if found and mode is not None:
            self._add(Task(TaskType.SETUP_PARALLEL_GROUP, mode, process_mode=TaskProcessMode.ALL_PROCESS))
        if rec.status == StrategyRecord.INIT:
            self._add(Task(TaskType.TUNE, rec.strategy, strategy_id=sid))
        self._add(Task(TaskType.DRYRUN, rec.strategy, strategy_id=sid, process_mode=TaskProcessMode.ALL_PROCESS))

    def _finish(self) -> None:
        ok = [r for r in self.strategies if r.status == StrategyRecord.SUCCEED]
        if ok:
            best = max(ok, key=lambda r: r.throughput)
            self._add(Task(TaskType.FINISH, best.strategy, process_mode=TaskProcessMode.ALL_PROCESS))
        else:
            self._add(Task(TaskType.FAIL, None, process_mode=TaskProcessMode.ALL_PROCESS))

    def _plan_more(self) -> None:
        """Called when the queue has drained and nothing is running."""
        if self.terminate_task_id is not None:
            return
        if self._candidates is None:
            self._generate_candidates()
        rec = self._next_candidate()
        if rec is None:
            self._finish()
        else:
            self._schedule_strategy(rec)

    # ------------------------------------------------------------------ worker-facing calls
    def get_task(self, process_id: int) -> Task:
        with self.lock:
            if self.assigning is None and self.busy.get(process_id) is None:
                while self.pending:
                    tid = self.pending[0]
                    t = self.tasks[tid]
                    if t.task_type == TaskType.SETUP_PARALLEL_GROUP and t.task_info == self.current_parallel_mode:
                        self.pending.popleft()          # this layout is already in place
                        t.status = TaskStatus.CANCELLED
                        continue
                    if t.process_mode == TaskProcessMode.ONE_PROCESS or self.total_process == 1:
                        if any(v is not None for v in self.busy.values()) and \
                                t.task_type in (TaskType.FINISH, TaskType.FAIL):
                            break
                        self.pending.popleft()
                        t.status = TaskStatus.RUNNING
                        t.process_assigned.append(process_id)
                        self.busy[process_id] = tid
                        return t
                    self.pending.popleft()
                    self.assigning, t.status = tid, TaskStatus.ASSIGNING
                    break
            if self.assigning is not None:
                t = self.tasks[self.assigning]
                all_idle = all(v is None for v in self.busy.values())
                if (t.process_assigned or all_idle) and process_id not in t.process_assigned \
                        and self.busy.get(process_id) is None:
                    t.process_assigned.append(process_id)
                    self.busy[process_id] = t.task_id
                    if len(t.process_assigned) == self.total_process:
                        self.assigning, t.status = None, TaskStatus.RUNNING
                    return t
            return Task(TaskType.WAIT)

    def report_task_result(self, task_id: int, process_id: int, status: bool, result=None) -> None:
        with self.lock:
            t = self.tasks[task_id]
            self.busy[process_id] = None
            t.reported.append(process_id)
            if t.process_mode == TaskProcessMode.ALL_PROCESS and self.total_process > 1:
                if process_id == 0:
                    t.task_result, t.status = result, (TaskStatus.SUCCEEDED if status else TaskStatus.FAILED)
                elif not status:
                    t.status = TaskStatus.FAILED
                if len(t.reported) < self.total_process:
                    return
                status = t.status != TaskStatus.FAILED
                result = t.task_result
            else:
                t.task_result, t.status = result, (TaskStatus.SUCCEEDED if status else TaskStatus.FAILED)
            self._task_done(t, status, result)
            if not self.pending and self.assigning is None and all(v is None for v in self.busy.values()):
                self._plan_more()

    def _task_done(self, t: Task, ok: bool, result) -> None:
        if t.task_type == TaskType.ANALYSE:
            if ok and isinstance(result, dict):
                self.analysis.update(result)
        elif t.task_type == TaskType.SETUP_PARALLEL_GROUP:
            if ok:
                self.current_parallel_mode = t.task_info
        elif t.task_type == TaskType.TUNE:
            rec = self.strategies[t.strategy_id]
            if ok:
                if result is not None:
                    rec.strategy = result if isinstance(result, Strategy) else Strategy(list(result))
                    for later in self.tasks.values():        # the dry run uses the tuned strategy
                        if later.strategy_id == t.strategy_id and later.task_type == TaskType.DRYRUN:
                            later.task_info = rec.strategy
                rec.status = StrategyRecord.TUNED
            else:
                rec.status = StrategyRecord.FAILED
                for later in self.tasks.values():
                    if later.strategy_id == t.strategy_id and later.task_id in self.pending:
                        self.pending.remove(later.task_id)
                        later.status = TaskStatus.CANCELLED
        elif t.task_type == TaskType.DRYRUN:
            rec = self.strategies[t.strategy_id]
            rec.dryrun_result = result if isinstance(result, dict) else {}
            rec.status = StrategyRecord.SUCCEED if (ok and rec.throughput > 0) else StrategyRecord.FAILED

    def best_strategy(self) -> Optional[Strategy]:
        ok = [r for r in self.strategies if r.status == StrategyRecord.SUCCEED]
        return max(ok, key=lambda r: r.throughput).strategy if ok else None
