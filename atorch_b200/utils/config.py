"""``Config``: attribute dictionary loadable from a python file (``Config.from_file("cfg.py")``) or a dict
(reference: atorch/utils/config.py:9-100)."""
from __future__ import annotations

import runpy
from typing import Any


class Config(dict):
    def __getattr__(self, k: str) -> Any:
        try:
            v = self[k]
        except KeyError as e:
            raise AttributeError(k) from e
        return Config(v) if isinstance(v, dict) and not isinstance(v, Config) else v

    def __setattr__(self, k: str, v: Any) -> None:
        self[k] = v

    @classmethod
    def from_file(cls, path: str) -> "Config":
        ns = runpy.run_path(path)
        return cls({k: v for k, v in ns.items() if not k.startswith("_") and not callable(v) and
                    not isinstance(v, type(runpy))})

    @classmethod
    def from_dict(cls, d: dict) -> "Config":
        return cls(d)

    def update_from(self, other: dict) -> "Config":
        for k, v in other.items():
            if isinstance(v, dict) and isinstance(self.get(k), dict):
                self[k] = Config(self[k]).update_from(v)
            else:
                self[k] = v
        return self
