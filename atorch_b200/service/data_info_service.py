"""Directory of produced batches: coworkers report ``(coworker_addr, batch_num)`` after they queue batches,
trainers ask which coworker to fetch the next batch from. Entries are handed out in arrival order, one
batch per answer. (Reference: atorch/service/data_info_service.py:15-64.)"""
from __future__ import annotations

import queue

from . import rpc

SERVICE = "atorch.DataInfoService"


class DataInfoServicer:
    def __init__(self, get_timeout: float = 60.0):
        self.queue: "queue.Queue[str]" = queue.Queue()
        self.get_timeout = get_timeout

    def report_data_info(self, info, context=None):
        for _ in range(int(info["batch_num"])):
            self.queue.put(info["coworker_addr"])
        return {}

    def get_data_info(self, request=None, context=None):
        try:
            return {"coworker_addr": self.queue.get(timeout=self.get_timeout)}
        except queue.Empty:
            return {"coworker_addr": None}


def create_data_info_service(port: int = 0, pool_size: int = 10):
    s = DataInfoServicer()
    return rpc.create_server(SERVICE, {"report_data_info": s.report_data_info, "get_data_info": s.get_data_info},
                             port, pool_size)
