"""Small gRPC toolkit shared by the services of this package: a server built from plain Python callables
registered as generic unary-unary handlers, and a client stub for them. Messages are pickled objects
(``cloudpickle`` when present, so functions defined in ``__main__`` or closures travel too); the message
size cap is 1 GiB as in the reference (atorch/common/constants.py:5-12). No generated ``*_pb2`` code."""
from __future__ import annotations

import pickle
from concurrent import futures
from typing import Callable, Dict, Optional

try:
    import cloudpickle as _cp
except ImportError:  # pragma: no cover
    _cp = pickle

MAX_MESSAGE = 1 << 30
OPTIONS = [("grpc.max_send_message_length", MAX_MESSAGE), ("grpc.max_receive_message_length", MAX_MESSAGE)]


def dumps(obj) -> bytes:
    return _cp.dumps(obj)


def loads(data: bytes):
    return pickle.loads(data)


def create_server(service: str, methods: Dict[str, Callable], port: int = 0, pool_size: int = 10,
                  host: str = "127.0.0.1"):
    """``methods``: name -> fn(request, context) -> response. Returns the started-less server with
    ``bound_port`` set; call ``.start()``."""
    import grpc

    server = grpc.server(futures.ThreadPoolExecutor(max_workers=pool_size), options=OPTIONS)
    handlers = {n: grpc.unary_unary_rpc_method_handler(fn, request_deserializer=loads, response_serializer=dumps)
                for n, fn in methods.items()}
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(service, handlers),))
    server.bound_port = server.add_insecure_port(f"{host}:{port}")
    return server


class Stub:
    def __init__(self, addr: str, service: str, timeout: Optional[float] = 300.0):
        import grpc

        self.addr, self.service, self.timeout = addr, service, timeout
        self.channel = grpc.insecure_channel(addr, options=OPTIONS)
        self._calls: Dict[str, Callable] = {}

    def call(self, method: str, request=None, timeout: Optional[float] = None):
        fn = self._calls.get(method)
        if fn is None:
            fn = self._calls[method] = self.channel.unary_unary(f"/{self.service}/{method}",
                                                                request_serializer=dumps, response_deserializer=loads)
        return fn(request, timeout=timeout or self.timeout)

    def close(self) -> None:
        self.channel.close()

    def __del__(self):
        try:
            self.channel.close()
        except Exception:  # noqa: BLE001
            pass
