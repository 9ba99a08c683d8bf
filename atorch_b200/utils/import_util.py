"""Import helpers and availability probes of optional packages.
(Reference: atorch/utils/import_util.py:13-170. Probes of back ends this framework does not target - NPU, XLA -
answer from the environment like the others and are False on a B200 box.)"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys


def import_module_from_py_file(file_path: str):
    name = os.path.splitext(os.path.basename(file_path))[0]
    spec = importlib.util.spec_from_file_location(name, file_path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def import_module(module_name: str):
    """``a.b.c`` -> attribute ``c`` of module ``a.b`` (or the module ``a.b.c`` itself)."""
    try:
        return importlib.import_module(module_name)
    except ImportError:
        parent, _, attr = module_name.rpartition(".")
        return getattr(importlib.import_module(parent), attr)


def _has(pkg: str) -> bool:
    try:
        return importlib.util.find_spec(pkg) is not None
    except (ImportError, ValueError):
        return False


def is_torch_npu_available(check_device: bool = False) -> bool:
    return _has("torch_npu")


def is_torch_xla_available() -> bool:
    return _has("torch_xla")


def is_xla_device_available() -> bool:
    return False


def is_triton_available() -> bool:
    return _has("triton")


def is_coverage_available() -> bool:
    return _has("coverage")


def is_megatron_lm_available() -> bool:
    return _has("megatron")


def is_flash_attn_3_avaliable(verbose: bool = False) -> bool:
    return _has("flash_attn_interface") or _has("flash_attn_3")


def is_liger_kernel_available() -> bool:
    return _has("liger_kernel")


def is_training_event_available() -> bool:
    return _has("dlrover")


def is_deep_gemm_available() -> bool:
    return _has("deep_gemm")


def is_native_kernels_available() -> bool:
    """The sm_100a kernel library of this package is loaded (a CUDA device is present)."""
    from .. import _lib

    return _lib.have_kernels()
