"""Sharded asynchronous checkpoint saver / loader of the engine-based trainer.

``FsdpShardCkptAsyncSaver.save(iteration, output_dir, train_args, module, optimizer, extra_state)`` writes
``output_dir/iter_{iteration:07d}/`` asynchronously (host staging + writer thread) and ``extra_state.pth``;
the tracker file moves only after all ranks finished. ``FsdpShardDcpCkptLoader.load`` restores the
iteration named by the tracker (the maximum over ranks).
(Reference: atorch/trainer/fsdp/fsdp_shard_async_saver.py:28-132, fsdp_shard_dcp_loader.py:19-91,
fsdp_ckpt_saver.py:9-64.)"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ...utils import fsdp_async_ckpt_util as A


@dataclass
class ExtraState:
    iteration: int = 0
    consumed_samples: int = 0
    lr_scheduler: Optional[dict] = None
    rng_state: Optional[dict] = None
    others: Dict[str, Any] = field(default_factory=dict)


class FsdpShardCkptAsyncSaver:
    def __init__(self, **kwargs):
        self.kwargs = kwargs

    def save(self, iteration: int, output_dir: str, train_args=None, module=None, optimizer=None,
             extra_state: Optional[ExtraState] = None, best_model_checkpoint=None, **_):
        extra = {"extra_state": extra_state.__dict__ if isinstance(extra_state, ExtraState) else (extra_state or {})}
        A.save_checkpoint(iteration, module, optimizer, output_dir, extra_sds=extra,
                          extra_paths={"extra_state": os.path.join(output_dir, f"iter_{iteration:07d}", "extra_state.pth")})

    def finish(self) -> None:
        A.wait_for_checkpoint()


class FsdpShardDcpCkptLoader:
    def load(self, resume_from_ckpt: str, model=None, optimizer=None, extra_state: Optional[ExtraState] = None,
             ckpt_step: Optional[int] = None, **_):
        step = ckpt_step if ckpt_step is not None else A.latest_checkpoint_step(resume_from_ckpt)
        if step is None:
            return None
        if dist.is_initialized():
            t = torch.tensor([step])
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            step = int(t.item())
        A.load_checkpoint(model, optimizer, resume_from_ckpt, step)
        f = os.path.join(resume_from_ckpt, f"iter_{step:07d}", "extra_state.pth")
        if os.path.exists(f):
            st = torch.load(f, weights_only=False)
            if isinstance(extra_state, ExtraState):
                extra_state.__dict__.update(st)
            return st
        return {"iteration": step}
