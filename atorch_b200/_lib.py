"""ctypes loader for ``libatb.so`` (the sm_100a kernels of atorch_b200).

The library is built in-tree by :mod:`atorch_b200.build`. On a machine with a GPU a missing
library is an error (ops must never fall back silently to eager PyTorch); on a CPU-only machine
``lib()`` returns ``None`` and the ops use their PyTorch reference implementations, which is what
the CPU test-suite exercises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent / "_C" / "libatb.so"
_lib = None
_tried = False


class KernelError(RuntimeError):
    """A launcher rejected its arguments or a kernel reported a non-zero status."""


launch_count = 0  # kernels of this library launched so far in this process
_NOT_LAUNCHES = {"atb_norm_bwd_parts", "atb_sumsq_parts", "atb_set_comm_wait_ns", "atb_noalloc_max_n"}


class _CountingLib:
    """Proxy over the ctypes library that counts kernel launches (one per launcher call)."""

    def __init__(self, cdll):
        self._cdll = cdll
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._cdll, name)
            if name in _NOT_LAUNCHES:
                fn = raw
            else:
                def fn(*a, _raw=raw):
                    global launch_count
                    launch_count += 1
                    return _raw(*a)
            self._cache[name] = fn
        return fn

    def has(self, name) -> bool:
        return hasattr(self._cdll, name)


def lib_path() -> Path:
    return _LIB_PATH


def lib():
    """The loaded library, or None on a CPU-only machine."""
    global _lib, _tried
    if _lib is not None:
        return _lib
    if not torch.cuda.is_available():
        return None
    if _tried:
        raise KernelError(f"{_LIB_PATH} could not be loaded")
    _tried = True
    if not _LIB_PATH.exists():
        if os.environ.get("ATB_AUTO_BUILD", "1") == "1":
            from . import build as _build

            _build.build()
        else:
            raise KernelError(f"{_LIB_PATH} is missing: run `python -m atorch_b200.build`")
    _lib = _CountingLib(ctypes.CDLL(str(_LIB_PATH)))
    return _lib


def have_kernels() -> bool:
    return lib() is not None


def use_kernels(*tensors: torch.Tensor) -> bool:
    """True when the CUDA kernels must be used for these tensors (all on a CUDA device)."""
    if not tensors or not all(t.is_cuda for t in tensors if t is not None):
        return False
    return lib() is not None


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what}: launcher returned {rc}")


_status: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write an error code to."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def check_status(device: torch.device) -> None:
    """Synchronising check of the status word; raises if a bounded wait ran out."""
    t = status_word(device)
    v = int(t.item())
    if v != 0:
        t.zero_()
        raise KernelError(f"kernel status {v} (1 = wait timeout, 3 = TMEM allocation, 4 = peer timeout)")


DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
