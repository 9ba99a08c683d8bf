"""Version probes: ``torch_version()`` as a comparable tuple and generic package-version comparisons.
(Reference: atorch/utils/version.py:13-80.)"""
from __future__ import annotations

import importlib
import re
from typing import Optional, Tuple


def get_digit_part(string: str) -> int:
    m = re.match(r"\d+", string)
    return int(m.group()) if m else 0


def _as_tuple(v) -> Tuple[int, ...]:
    if isinstance(v, (tuple, list)):
        return tuple(int(x) for x in v)
    return tuple(get_digit_part(p) for p in str(v).split("+")[0].split(".")[:3])


def torch_version(version: Optional[str] = None) -> Tuple[int, ...]:
    import torch

    return _as_tuple(version if version is not None else torch.__version__)


def get_version(package: str) -> Optional[Tuple[int, ...]]:
    try:
        from importlib.metadata import version as _v

        return _as_tuple(_v(package))
    except Exception:
        try:
            return _as_tuple(getattr(importlib.import_module(package), "__version__"))
        except Exception:
            return None


def package_version_smaller_than(pkg_name: str, version, print_version: bool = False) -> bool:
    v = get_version(pkg_name)
    if print_version:
        print(f"{pkg_name} version: {v}")
    return v is not None and v < _as_tuple(version)


def package_version_bigger_than(pkg_name: str, version) -> bool:
    v = get_version(pkg_name)
    return v is not None and v > _as_tuple(version)


def package_version_equal_to(pkg_name: str, version) -> bool:
    v = get_version(pkg_name)
    want = _as_tuple(version)
    return v is not None and v[: len(want)] == want


def get_megatron_version():
    return get_version("megatron-core") or get_version("megatron")


def is_megatron_version_bigger_than(version, check_equality: bool = True) -> bool:
    v = get_megatron_version()
    if v is None:
        return False
    return v >= _as_tuple(version) if check_equality else v > _as_tuple(version)
