"""Services a coworker (a CPU-only helper process) runs.

* ``CoworkerRpcService.get_batch_data``: hands out batches a coworker has produced into a queue (pull model:
  the coworker runs the whole input pipeline and trainers fetch finished batches).
* ``CoworkerRpcService.process``: runs ``fn`` over a list of items and returns the results (push model: the
  trainer's dataloader worker sends ``num_rpc_fuse`` items per call).

(Reference: atorch/service/coworker_data_service.py:16-70, protos/coworker.proto; the push model is served by
torch RPC in the reference, atorch/data/coworker_dataset.py:194-222.)"""
from __future__ import annotations

import queue
from typing import Optional

from . import rpc

SERVICE = "atorch.CoworkerRpcService"


class CoworkerRpcServicer:
    def __init__(self, batched_data_queue: Optional["queue.Queue"] = None, get_timeout: float = 60.0):
        self.queue = batched_data_queue
        self.get_timeout = get_timeout

    def get_batch_data(self, request, context=None):
        if self.queue is None:
            return {"data": None, "empty": True}
        try:
            return {"data": self.queue.get(timeout=self.get_timeout), "empty": False}
        except queue.Empty:
            return {"data": None, "empty": True}

    def process(self, request, context=None):
        fn, items = request["fn"], request["items"]
        out = []
        for it in items:
            try:
                out.append(fn(it))
            except Exception:  # noqa: BLE001 - a sample that fails to preprocess is reported as None
                out.append(None)
        return {"results": out}

    def ping(self, request, context=None):
        return {"ok": True}


def create_coworker_rpc_service(port: int = 0, data_queue: Optional["queue.Queue"] = None, pool_size: int = 8):
    s = CoworkerRpcServicer(data_queue)
    return rpc.create_server(SERVICE, {"get_batch_data": s.get_batch_data, "process": s.process, "ping": s.ping},
                             port, pool_size)


def run_coworker(port: int = 0, data_queue=None, ready=None, stop=None) -> None:
    """Serve until ``stop`` (a ``threading.Event`` / ``multiprocessing.Event``) is set. ``ready`` (a queue or
    pipe end with ``put``/``send``) receives the bound port."""
    server = create_coworker_rpc_service(port, data_queue)
    server.start()
    if ready is not None:
        (ready.put if hasattr(ready, "put") else ready.send)(server.bound_port)
    if stop is None:
        server.wait_for_termination()
    else:
        stop.wait()
        server.stop(None)
