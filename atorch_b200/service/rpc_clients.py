"""Clients of the data services. (Reference: atorch/service/rpc_clients.py:15-107.)"""
from __future__ import annotations

from typing import Dict, List

from . import coworker_data_service, data_info_service, rpc


class GpuPodRpcClient:
    """Used by a coworker to tell a trainer-side directory that batches are ready."""

    def __init__(self, grpc_addr: str):
        self.stub = rpc.Stub(grpc_addr, data_info_service.SERVICE)

    def report_data_info(self, coworker_addr: str, batch_num: int) -> None:
        self.stub.call("report_data_info", {"coworker_addr": coworker_addr, "batch_num": batch_num})


class DataInfoRpcClient:
    def __init__(self, grpc_addr: str):
        self.stub = rpc.Stub(grpc_addr, data_info_service.SERVICE)

    def get_data_info(self):
        return self.stub.call("get_data_info", {})["coworker_addr"]


class CoworkerRpcClient:
    def __init__(self, grpc_addr: str):
        self.addr = grpc_addr
        self.stub = rpc.Stub(grpc_addr, coworker_data_service.SERVICE)

    def get_batch_data(self):
        r = self.stub.call("get_batch_data", {})
        return None if r["empty"] else r["data"]

    def process(self, fn, items: List):
        return self.stub.call("process", {"fn": fn, "items": list(items)})["results"]

    def ping(self, timeout: float = 5.0) -> bool:
        try:
            return bool(self.stub.call("ping", {}, timeout=timeout)["ok"])
        except Exception:  # noqa: BLE001
            return False


def create_gpu_pod_rpc_clients(gpu_pod_addrs: List[str]) -> List[GpuPodRpcClient]:
    return [GpuPodRpcClient(a) for a in gpu_pod_addrs]


def create_data_info_rpc_client(addr: str) -> DataInfoRpcClient:
    return DataInfoRpcClient(addr)


def create_coworker_rpc_client(coworker_addrs: List[str]) -> Dict[str, CoworkerRpcClient]:
    return {a: CoworkerRpcClient(a) for a in coworker_addrs}
