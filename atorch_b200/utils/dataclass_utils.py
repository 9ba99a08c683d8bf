"""Helpers for argument dataclasses: JSON-friendly dumps, "only what differs from the defaults", mapping between two
naming schemes of the same options, and dataclasses that accept (and remember) unknown keyword arguments.
(Reference: atorch/utils/dataclass_utils.py:13-182.)
"""
from __future__ import annotations

import copy
import json
import logging
import os
from contextlib import contextmanager
from dataclasses import dataclass, field, fields
from enum import Enum

logger = logging.getLogger(__name__)


@contextmanager
def clear_environment():
    """An empty ``os.environ`` inside the block (defaults that read the environment show their plain values); the
    previous environment comes back afterwards."""
    saved = os.environ.copy()
    os.environ.clear()
    try:
        yield
    finally:
        os.environ.clear()
        os.environ.update(saved)


def is_json_serializable(obj) -> bool:
    try:
        json.dumps(obj)
        return True
    except (TypeError, OverflowError):
        return False


def _name_of(v) -> str:
    return v.__name__ if hasattr(v, "__name__") else str(v)


def _plain(d: dict) -> dict:
    """Values made JSON-friendly: callables by name, sequences of enums by value, nested dicts recursively, anything
    else that json cannot dump by name or ``str``."""
    out = {}
    for k, v in d.items():
        if callable(v):
            out[k] = _name_of(v)
        elif isinstance(v, (list, tuple)) and len(v) > 0 and isinstance(v[0], Enum):
            out[k] = type(v)(x.value for x in v)
        elif isinstance(v, (list, tuple)) and len(v) > 0 and callable(v[0]):
            out[k] = type(v)(_name_of(x) for x in v)
        elif isinstance(v, dict):
            out[k] = _plain(v)
        elif is_json_serializable(v):
            out[k] = v
        else:
            out[k] = _name_of(v)
    return out


class DataclassMixin:
    def to_dict(self) -> dict:
        """The ``init`` fields, JSON-friendly; an ``Enum`` field is given by its value."""
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.init}
        d = {k: (v.value if isinstance(v, Enum) else v) for k, v in d.items()}
        return _plain(d)

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2)

    def to_kwargs(self) -> dict:
        """Only the fields whose value differs from a default-constructed instance (built under an empty
        environment, so environment-driven defaults do not hide a difference)."""
        with clear_environment():
            defaults = self.__class__().to_dict()
        return {k: v for k, v in self.to_dict().items() if defaults[k] != v}


@dataclass
class AutoMapperExtraConfigs:
    """``extra_configs`` carries options under another system's names. ``do_auto_mapping({own: other})`` fills the
    other names from the own fields; where both are set and differ the other name wins (and the own field is updated,
    with a warning)."""

    extra_configs: dict = field(default_factory=dict)

    def do_auto_mapping(self, name_map: dict, overwrite_extra_configs: bool = False) -> dict:
        target = self.extra_configs if overwrite_extra_configs else copy.copy(self.extra_configs)
        for own, other in name_map.items():
            mine = getattr(self, own)
            if other not in target or (target[other] is None and mine is not None):
                target[other] = mine
            elif target[other] != mine:
                logger.warning("%s:%s will be overridden by %s:%s", own, mine, other, target[other])
                setattr(self, own, target[other])
        return target


@dataclass
class DynamicDataClass(DataclassMixin):
    """Base for dataclasses built from loosely specified keyword arguments: declared fields are set from the
    arguments or their class-level defaults (a field with neither is an error); unknown arguments are kept, readable as
    attributes and included in ``to_dict()``."""

    def __init__(self, **kwargs):
        names = {f.name for f in fields(self)}
        for name in names:
            if name in kwargs:
                setattr(self, name, kwargs[name])
            elif not hasattr(type(self), name):
                raise ValueError(f"{name} is not found in __init__ params and has no default value")
            else:
                setattr(self, name, getattr(self, name))
        object.__setattr__(self, "_additional_data", {k: copy.deepcopy(v) for k, v in kwargs.items() if k not in names})

    def to_dict(self) -> dict:
        d = super().to_dict()
        d.update(self._additional_data)
        return d

    def __getattr__(self, item):
        extra = self.__dict__.get("_additional_data", {})
        if item in extra:
            return extra[item]
        raise AttributeError(f"'{self.__class__.__name__}' object has no attribute '{item}'")
