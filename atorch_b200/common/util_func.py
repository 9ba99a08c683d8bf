"""Small helpers (reference: atorch/common/util_func.py): device moves of nested batches, free ports,
recursive attribute access, integer division checks."""
from __future__ import annotations

import socket

import torch


def data_to_device(data, device, non_blocking: bool = True):
    if isinstance(data, torch.Tensor):
        return data.to(device, non_blocking=non_blocking)
    if isinstance(data, dict):
        return {k: data_to_device(v, device, non_blocking) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(data_to_device(v, device, non_blocking) for v in data)
    return data


def data_float_to_dtype(data, dtype):
    if isinstance(data, torch.Tensor):
        return data.to(dtype) if data.is_floating_point() else data
    if isinstance(data, dict):
        return {k: data_float_to_dtype(v, dtype) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(data_float_to_dtype(v, dtype) for v in data)
    return data


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def recursively_getattr(obj, name: str):
    for part in name.split("."):
        obj = getattr(obj, part)
    return obj


def recursively_setattr(obj, name: str, value) -> None:
    parts = name.split(".")
    for part in parts[:-1]:
        obj = getattr(obj, part)
    setattr(obj, parts[-1], value)


def divide(a: int, b: int) -> int:
    assert a % b == 0, f"{a} is not divisible by {b}"
    return a // b
