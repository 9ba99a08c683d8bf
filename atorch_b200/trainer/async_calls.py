"""Asynchronous calls with distributed finalisation (the machinery behind asynchronous checkpoint saves).

``AsyncRequest``        what to run in the background (``async_fn(*args)``) and what to run afterwards on every rank
                        (``finalize_fns``), once the background part has finished *on all ranks*.
``DistributedAsyncCaller``  runs one such call in a forked process or in a thread and answers "is it done
                        everywhere?" with a single two-integer all-reduce (alive count, failure count). A call that
                        outlives its timeout is terminated and counted as failed.
``AsyncCallsQueue``     any number of calls in flight, finalised strictly in order.
``AsyncCheckpointSaver``  the saver built on them: write the rank's files in the background, then - when every rank
                        has written - run the finalisation (tracker file) once.

The reductions run on the default process group's device (CPU tensors for gloo), so the module works without a GPU.
(Reference: atorch/trainer/base/dist_checkpointing/strategies/async_utils.py:30-357 and
atorch/trainer/megatron/megatron_async_save.py:81-244; the Megatron-specific state-dict preparation has no
counterpart here, the saver takes any ``write_fn``.)
"""
from __future__ import annotations

import logging
import multiprocessing as mp
import os
import threading
import time
import traceback
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, List, Optional, Tuple

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)


@dataclass
class AsyncRequest:
    async_fn: Optional[Callable]
    async_fn_args: Tuple = ()
    finalize_fns: List[Callable] = field(default_factory=list)
    is_frozen: bool = False

    def add_finalize_fn(self, fn: Callable) -> None:
        """Appended after the existing ones; refused once the request is frozen (scheduled)."""
        if self.is_frozen:
            raise RuntimeError("Cannot add finalization functions to a frozen AsyncRequest")
        self.finalize_fns.append(fn)

    def execute_sync(self) -> None:
        """The same effects without any background work: run, wait for all ranks, finalise."""
        if self.async_fn is not None:
            self.async_fn(*self.async_fn_args)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        for fn in self.finalize_fns:
            fn()

    def freeze(self) -> "AsyncRequest":
        return AsyncRequest(self.async_fn, self.async_fn_args, list(self.finalize_fns), True)


def _reduce_pair(alive: int, failed: int) -> Tuple[int, int]:
    """Sum of (alive, failed) over the ranks; the cost of a barrier."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return alive, failed
    dev = "cuda" if dist.get_backend() == "nccl" and torch.cuda.is_available() else "cpu"
    t = torch.tensor([alive, failed], dtype=torch.int32, device=dev)
    dist.all_reduce(t)
    return int(t[0]), int(t[1])


def _run_guarded(fn: Callable, args: Tuple, fail_flag) -> None:
    try:
        fn(*args)
    except BaseException:      # the parent must learn of any failure, also SystemExit in a child process
        traceback.print_exc()
        fail_flag.value = 1


class DistributedAsyncCaller:
    """One background call at a time. ``mode="process"`` forks (the call sees a snapshot of this process's memory, so
    tensors staged on the host need no copy); ``mode="thread"`` shares the address space. Every method is collective:
    call it on all ranks."""

    def __init__(self, mode: str = "process", timeout: float = 20 * 60):
        assert mode in ("process", "thread"), mode
        self.mode, self.timeout = mode, timeout
        self.worker = None
        self.start_time: Optional[float] = None
        self._fail = None
        self.is_fail = 0

    def schedule_async_call(self, async_fn: Optional[Callable], save_args: Tuple = (), timeout: Optional[float] = None):
        if async_fn is None:
            return
        assert self.worker is None, "the previous call has not been finalised"
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.synchronize()            # whatever the call reads has been produced
        if timeout is not None:
            self.timeout = timeout
        self.is_fail = 0
        self.start_time = time.time()
        if self.mode == "process":
            ctx = mp.get_context("fork")
            self._fail = ctx.Value("i", 0)
            self.worker = ctx.Process(target=_run_guarded, args=(async_fn, tuple(save_args), self._fail), daemon=True)
        else:
            self._fail = _Flag()
            self.worker = threading.Thread(target=_run_guarded, args=(async_fn, tuple(save_args), self._fail),
                                           daemon=True)
        self.worker.start()

    def _local_state(self) -> Tuple[int, int]:
        alive = int(self.worker.is_alive()) if self.worker is not None else 0
        if alive and self.mode == "process" and time.time() - self.start_time > self.timeout:
            logger.warning("async call exceeded its %.0f s timeout on rank %s: terminated", self.timeout,
                           os.environ.get("RANK", "0"))
            self.worker.terminate()
            self.worker.join()
            self.worker, alive, self.is_fail = None, 0, 1
        if self.worker is not None and not alive:
            if self._fail is not None and self._fail.value:
                self.is_fail = 1
            if self.mode == "process" and self.worker.exitcode not in (0, None):
                self.is_fail = 1
        return alive, self.is_fail

    def is_current_async_call_done(self, blocking: bool = False) -> Tuple[bool, bool]:
        """``(done on all ranks, failed on some rank)``. Non-blocking: returns at once while any rank still works.
        Blocking: joins the local call, then agrees with the other ranks."""
        alive, failed = _reduce_pair(*self._local_state())
        if alive > 0 and not blocking:
            return False, failed > 0
        if self.worker is not None:
            self.worker.join(None if self.mode == "thread" else max(self.timeout - (time.time() - self.start_time), 0))
        alive, failed = _reduce_pair(*self._local_state())
        while alive > 0 and blocking:           # another rank is slower: poll at barrier cost
            time.sleep(0.05)
            alive, failed = _reduce_pair(*self._local_state())
        if alive == 0:
            self.worker, self.start_time = None, None
        return alive == 0, failed > 0

    def close(self) -> None:
        if self.worker is not None:
            if self.mode == "process" and self.worker.is_alive():
                self.worker.terminate()
            self.worker.join()
            self.worker = None


class _Flag:
    value = 0


class AsyncCallsQueue:
    """Several asynchronous requests in flight, finalised in the order they were scheduled."""

    def __init__(self, mode: str = "process", timeout: float = 20 * 60):
        self.mode, self.timeout = mode, timeout
        self.calls: Deque[Tuple[int, DistributedAsyncCaller, AsyncRequest]] = deque()
        self.call_idx = -1
        self.failed: List[int] = []

    def schedule_async_request(self, request: AsyncRequest) -> int:
        self.call_idx += 1
        caller = DistributedAsyncCaller(self.mode, self.timeout)
        request = request.freeze()
        caller.schedule_async_call(request.async_fn, request.async_fn_args)
        self.calls.append((self.call_idx, caller, request))
        return self.call_idx

    def maybe_finalize_async_calls(self, blocking: bool = False) -> List[int]:
        """Finalise the oldest calls that are done on all ranks (all of them when ``blocking``); returns their
        indices. The finalisation functions of a call that failed on some rank are not run: its index goes to
        ``self.failed`` on every rank."""
        finalized = []
        while self.calls:
            idx, caller, request = self.calls[0]
            done, failed = caller.is_current_async_call_done(blocking)
            if not done:
                break
            self.calls.popleft()
            if failed:
                logger.error("asynchronous call %d failed on some rank: not finalised", idx)
                self.failed.append(idx)
            else:
                for fn in request.finalize_fns:
                    fn()
            finalized.append(idx)
        return finalized

    def get_num_unfinalized_calls(self) -> int:
        return len(self.calls)

    def close(self) -> None:
        self.maybe_finalize_async_calls(blocking=True)


class AsyncCheckpointSaver:
    """Checkpoint saves that do not hold up training: ``save(iteration, write_fn, args)`` starts ``write_fn(*args)``
    in the background on every rank (a fork sees the host-staged state as it is now) and returns; a later
    ``maybe_finalize()`` - call it every step - notices when all ranks have written and then, on rank 0, records the
    iteration in the tracker file ``latest_checkpointed_iteration.txt`` of ``root``."""

    TRACKER = "latest_checkpointed_iteration.txt"

    def __init__(self, root: str, mode: str = "process", timeout: float = 20 * 60, max_in_flight: int = 1):
        self.root, self.max_in_flight = root, max_in_flight
        self.queue = AsyncCallsQueue(mode, timeout)

    def save(self, iteration: int, write_fn: Callable, args: Tuple = (), extra_finalize: Optional[Callable] = None) -> int:
        while self.queue.get_num_unfinalized_calls() >= self.max_in_flight:
            self.queue.maybe_finalize_async_calls(blocking=True)
        req = AsyncRequest(write_fn, tuple(args), [])
        req.add_finalize_fn(lambda: self._write_tracker(iteration))
        if extra_finalize is not None:
            req.add_finalize_fn(extra_finalize)
        return self.queue.schedule_async_request(req)

    def _write_tracker(self, iteration: int) -> None:
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        if rank == 0:
            os.makedirs(self.root, exist_ok=True)
            tmp = os.path.join(self.root, self.TRACKER + ".tmp")
            with open(tmp, "w") as f:
                f.write(str(iteration))
            os.replace(tmp, os.path.join(self.root, self.TRACKER))

    def maybe_finalize(self, blocking: bool = False) -> List[int]:
        return self.queue.maybe_finalize_async_calls(blocking)

    def latest_iteration(self) -> Optional[int]:
        p = os.path.join(self.root, self.TRACKER)
        return int(open(p).read().strip()) if os.path.exists(p) else None

    def close(self) -> None:
        self.queue.close()
