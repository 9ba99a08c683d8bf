"""The acceleration engine as a network service: rank 0 runs ``AccelerationEngine`` (an ``Executor`` behind a
gRPC server), every rank's ``AutoAccelerationClient`` loops ``get_task`` → run → ``report_task_result``.

The two RPCs (``/atorch.AutoAccelerationService/get_task`` and ``.../report_task_result``) are registered
as generic unary-unary handlers whose messages are pickled Python dicts, so no generated stubs are needed;
the message fields follow the reference's ``acceleration.proto`` (task_id, task_type, process_mode,
time_limit, strategy / analysis_method / parallel_group_info; process_id, status, result).
(Reference: atorch/auto/engine/acceleration_engine.py:11-96, servicer.py:17-80, client.py:35-93,
atorch/protos/acceleration.proto.)
"""
from __future__ import annotations

import os
import pickle
import time
from concurrent import futures
from typing import Optional

from ...common.log_utils import default_logger as logger
from .executor import Executor
from .task import Task, TaskType

SERVICE = "atorch.AutoAccelerationService"
MAX_MESSAGE = 1 << 30        # strategies carry configs with classes and small tensors; same cap as the reference


def _task_message(t: Task) -> dict:
    return {"task_id": t.task_id, "task_type": t.task_type, "process_mode": t.process_mode,
            "time_limit": t.time_limit, "task_info": t.task_info}


class AutoAccelerationService:
    def __init__(self, executor: Executor):
        self.executor = executor

    def get_task(self, request: dict, context=None) -> dict:
        return _task_message(self.executor.get_task(int(request["process_id"])))

    def report_task_result(self, request: dict, context=None) -> dict:
        self.executor.report_task_result(int(request["task_id"]), int(request["process_id"]),
                                         bool(request["status"]), request.get("result"))
        return {}


def create_acceleration_service(port: int, executor: Executor, pool_size: Optional[int] = None):
    import grpc

    pool_size = pool_size or int(os.getenv("WORLD_SIZE", "8"))
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=pool_size),
                         options=[("grpc.max_send_message_length", MAX_MESSAGE),
                                  ("grpc.max_receive_message_length", MAX_MESSAGE)])
    svc = AutoAccelerationService(executor)
    handlers = {name: grpc.unary_unary_rpc_method_handler(fn, request_deserializer=pickle.loads,
                                                          response_serializer=pickle.dumps)
                for name, fn in (("get_task", svc.get_task), ("report_task_result", svc.report_task_result))}
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(SERVICE, handlers),))
    bound = server.add_insecure_port(f"127.0.0.1:{port}" if os.getenv("ATORCH_ENGINE_LOCAL_ONLY", "1") == "1"
                                     else f"[::]:{port}")
    server.bound_port = bound
    return server


class AccelerationEngine:
    def __init__(self, device_context=None, included_opts=None, excluded_opts=None, time_limit=None,
                 load_strategy=None, verbose: bool = False, algo: str = "combination"):
        self.executor = Executor(device_context, included_opts, excluded_opts, time_limit, load_strategy, algo,
                                 verbose)
        self.port: Optional[int] = None
        self.service = None

    def start_service(self, port: int = 0) -> int:
        self.service = create_acceleration_service(port, self.executor)
        self.service.start()
        self.port = self.service.bound_port
        logger.info(f"auto-acceleration service listening on port {self.port}")
        return self.port

    def tear_down(self, force_stopping: bool = False, timeout: float = 120.0) -> None:
        t0 = time.time()
        while not self.executor.can_be_terminated and not force_stopping and time.time() - t0 < timeout:
            time.sleep(0.05)
        if not self.executor.can_be_terminated:
            logger.warning("not every process received the terminating task")
        if self.service is not None:
            self.service.stop(None)

    def service_port(self) -> Optional[int]:
        return self.port


class AutoAccelerationClient:
    def __init__(self, addr: str, process_id: int):
        import grpc

        self.process_id = process_id
        self.channel = grpc.insecure_channel(addr, options=[("grpc.max_send_message_length", MAX_MESSAGE),
                                                            ("grpc.max_receive_message_length", MAX_MESSAGE)])
        self._get = self.channel.unary_unary(f"/{SERVICE}/get_task", request_serializer=pickle.dumps,
                                             response_deserializer=pickle.loads)
        self._report = self.channel.unary_unary(f"/{SERVICE}/report_task_result", request_serializer=pickle.dumps,
                                                response_deserializer=pickle.loads)

    def get_task(self) -> Task:
        m = self._get({"process_id": self.process_id}, timeout=60)
        t = Task(m["task_type"], m["task_info"], task_id=m["task_id"], process_mode=m["process_mode"],
                 time_limit=m["time_limit"])
        return t

    def report_task_result(self, task: Task, status: bool, result=None) -> None:
        self._report({"task_id": task.task_id, "process_id": self.process_id, "status": status,
                      "task_type": task.task_type, "result": result}, timeout=60)

    def close(self) -> None:
        self.channel.close()


def run_worker_loop(client: AutoAccelerationClient, run_task, poll_interval: float = 0.05):
    """``run_task(task) -> (ok, result)`` for ANALYSE / SETUP_PARALLEL_GROUP / TUNE / DRYRUN. Returns the
    final strategy (FINISH) or None (FAIL)."""
    while True:
        task = client.get_task()
        if task.task_type == TaskType.WAIT:
            time.sleep(poll_interval)
            continue
        if task.task_type in (TaskType.FINISH, TaskType.FAIL):
            client.report_task_result(task, task.task_type == TaskType.FINISH, None)
            return task.task_info if task.task_type == TaskType.FINISH else None
        try:
            ok, result = run_task(task)
        except Exception as e:  # noqa: BLE001 - a failing candidate is a result, not the end of the search
            logger.warning(f"task {task.task_type} failed: {e}")
            ok, result = False, None
        client.report_task_result(task, ok, result)
