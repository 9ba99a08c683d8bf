"""Per-stage checkpoints of a pipeline job: every pipe rank saves / loads the chunks it owns under
``{dir}/pipe_stage_{stage_id:03d}.pt`` (plus its optimizer state).
(Reference: atorch/utils/pipe_file_utils.py:41-113.)"""
from __future__ import annotations

import os

import torch

from ..distributed import distributed as D


def atorch_save_pipe_checkpoint(pipe_module, path: str, optimizer=None, only_data_rank0: bool = True) -> None:
    os.makedirs(path, exist_ok=True)
    if only_data_rank0 and (D.parallel_rank("data") or 0) != 0:
        return
    for m, sid in zip(pipe_module.stage_modules, pipe_module.stage_ids):
        inner = m.module if hasattr(m, "module") and isinstance(m.module, torch.nn.Module) else m
        torch.save(inner.state_dict(), os.path.join(path, f"pipe_stage_{sid:03d}.pt"))
    if optimizer is not None:
        torch.save(optimizer.state_dict(), os.path.join(path, f"pipe_optim_{pipe_module.pp_rank:03d}.pt"))


def atorch_load_pipe_checkpoint(pipe_module, path: str, optimizer=None, strict: bool = True) -> None:
    for m, sid in zip(pipe_module.stage_modules, pipe_module.stage_ids):
        inner = m.module if hasattr(m, "module") and isinstance(m.module, torch.nn.Module) else m
        inner.load_state_dict(torch.load(os.path.join(path, f"pipe_stage_{sid:03d}.pt"), map_location="cpu"),
                              strict=strict)
    f = os.path.join(path, f"pipe_optim_{pipe_module.pp_rank:03d}.pt")
    if optimizer is not None and os.path.exists(f):
        optimizer.load_state_dict(torch.load(f, map_location="cpu"))
