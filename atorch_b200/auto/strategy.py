"""``Strategy``: an ordered list of ``(optimisation name, config, tunable)`` entries.

Same role and pickle-file interchange as atorch/auto/strategy.py:4-128 of the reference.
"""
from __future__ import annotations

import pickle
from typing import Any, Iterator, List, Optional, Tuple


class Strategy:
    def __init__(self, opt_list: Optional[List[Tuple[str, Any, Optional[bool]]]] = None):
        self.opt_list: List[list] = [list(o) for o in (opt_list or [])]

    # container protocol -------------------------------------------------------------------------
    def __len__(self) -> int:
        return len(self.opt_list)

    def __iter__(self) -> Iterator:
        return iter(self.opt_list)

    def __getitem__(self, i):
        return self.opt_list[i]

    def __repr__(self) -> str:
        return "Strategy(" + ", ".join(f"{n}" for n, _, _ in self.opt_list) + ")"

    def __str__(self) -> str:
        return "\n".join(f"{n}: config={c!r} tunable={t}" for n, c, t in self.opt_list)

    def add_opt(self, opt) -> None:
        name, config, tunable = (list(opt) + [None, None])[:3]
        self.opt_list.append([name, config, tunable])

    def names(self) -> List[str]:
        return [o[0] for o in self.opt_list]

    def get(self, name: str):
        for o in self.opt_list:
            if o[0] == name:
                return o
        return None

    def is_tunable(self) -> bool:
        return any(bool(o[2]) for o in self.opt_list)

    def reset_config(self) -> None:
        for o in self.opt_list:
            if o[2]:
                o[1] = None

    def set_tunable_value(self, opt_lib) -> None:
        for o in self.opt_list:
            if o[2] is None:
                o[2] = bool(opt_lib[o[0]].is_tunable) and o[1] is None

    # parallel mode ------------------------------------------------------------------------------
    def get_parallel_mode(self):
        """(found, config): whether a ``parallel_mode`` entry exists and its config (may be None)."""
        o = self.get("parallel_mode")
        return (True, o[1]) if o is not None else (False, None)

    def adjust_data_parallel(self, size: int) -> None:
        o = self.get("parallel_mode")
        if o is None:
            return
        if o[1] is None:
            o[1] = ([("data", size)], None)
            return
        cfg = list(o[1])
        dims, found = [], False
        for n, s in cfg[0]:
            if n == "data":
                dims.append((n, size))
                found = True
            else:
                dims.append((n, s))
        if not found:
            dims.append(("data", size))
        cfg[0] = dims
        o[1] = tuple(cfg)

    def remove_distributed_method(self, opt_lib):
        removed = [o[0] for o in self.opt_list if opt_lib[o[0]].distributed_only(o[1])]
        self.opt_list = [o for o in self.opt_list if o[0] not in removed]
        return removed or None

    def remove_device_unsupported_method(self, opt_lib, device_capability):
        removed = [o[0] for o in self.opt_list if not opt_lib[o[0]].device_supported(o[1], device_capability)]
        self.opt_list = [o for o in self.opt_list if o[0] not in removed]
        return removed or None

    # persistence ----------------------------------------------------------------------------------
    def dumps(self) -> bytes:
        return pickle.dumps(self)

    @staticmethod
    def loads(data: bytes) -> "Strategy":
        s = pickle.loads(data)
        if not isinstance(s, Strategy):
            raise TypeError("not a pickled Strategy")
        return s
