"""Module-level numeric comparison between two runs: ``module_numeric_checker(model, dir, "save")``
registers hooks that dump every module's forward output; in ``"compare"`` mode the outputs are compared
with the dump and mismatches are reported with their max abs / rel error.
(Reference: atorch/utils/numberic_checker.py:54-150.)"""
from __future__ import annotations

import os
from typing import Dict, List

import torch
import torch.nn as nn


def _first_tensor(out):
    if isinstance(out, torch.Tensor):
        return out
    if isinstance(out, (tuple, list)):
        for o in out:
            t = _first_tensor(o)
            if t is not None:
                return t
    if isinstance(out, dict):
        for o in out.values():
            t = _first_tensor(o)
            if t is not None:
                return t
    return None


class module_numeric_checker:
    def __init__(self, model: nn.Module, path: str, mode: str = "save", rtol: float = 1e-3, atol: float = 1e-5):
        assert mode in ("save", "compare")
        self.model, self.path, self.mode, self.rtol, self.atol = model, path, mode, rtol, atol
        os.makedirs(path, exist_ok=True)
        self.mismatches: List[Dict] = []
        self.hooks = []
        self.calls: Dict[str, int] = {}

    def __enter__(self):
        for name, m in self.model.named_modules():
            self.hooks.append(m.register_forward_hook(self._hook(name or "root")))
        return self

    def __exit__(self, *exc):
        for h in self.hooks:
            h.remove()
        return False

    def _hook(self, name):
        def fn(mod, inp, out):
            t = _first_tensor(out)
            if t is None:
                return
            i = self.calls.get(name, 0)
            self.calls[name] = i + 1
            f = os.path.join(self.path, f"{name}.{i}.pt")
            if self.mode == "save":
                torch.save(t.detach().float().cpu(), f)
            elif os.path.exists(f):
                ref = torch.load(f)
                cur = t.detach().float().cpu()
                if ref.shape != cur.shape or not torch.allclose(cur, ref, rtol=self.rtol, atol=self.atol):
                    err = (cur - ref).abs().max().item() if ref.shape == cur.shape else float("inf")
                    self.mismatches.append({"module": name, "call": i, "max_abs_err": err})
        return fn


module_numberic_checker = module_numeric_checker   # the reference's spelling
