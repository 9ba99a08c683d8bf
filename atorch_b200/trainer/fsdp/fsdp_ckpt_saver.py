"""Sharded asynchronous checkpoint saver / loader of the engine-based trainer.

``FsdpShardCkptAsyncSaver.save(iteration, output_dir, train_args, module, optimizer, extra_state)`` writes
``output_dir/iter_{iteration:07d}/`` in the ``torch.distributed.checkpoint`` format (``.metadata`` +
``__{rank}_0.distcp``, state key ``"atorch_FsdpShardDcpCkpt"``; ``utils/dcp_io.py``) from host copies of the
shards on a writer thread, plus ``extra_state.pth``; ``finish()`` joins the writer, waits for every rank and
only then moves the tracker file. ``FsdpShardDcpCkptLoader.load`` restores the iteration named by the
tracker (the maximum over ranks) at any world size; directories written in the flat shard format
(``flat_param.*``) are still read.
(Reference: atorch/trainer/fsdp/fsdp_shard_async_saver.py:28-132, fsdp_shard_dcp_loader.py:19-91,
fsdp_ckpt_saver.py:9-64.)"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ...utils import dcp_io
from ...utils import fsdp_async_ckpt_util as A


@dataclass
class ExtraState:
    iteration: int = 0
    consumed_samples: int = 0
    lr_scheduler: Optional[dict] = None
    rng_state: Optional[dict] = None
    others: Dict[str, Any] = field(default_factory=dict)


class FsdpShardCkptAsyncSaver:
    def __init__(self, async_save: bool = True, **kwargs):
        self.async_save, self.kwargs = async_save, kwargs
        self._pending = None          # (iteration, output_dir) whose tracker has not moved yet

    def save(self, iteration: int, output_dir: str, train_args=None, module=None, optimizer=None,
             extra_state: Optional[ExtraState] = None, best_model_checkpoint=None, **_):
        self.finish()
        d = os.path.join(output_dir, f"iter_{iteration:07d}")
        os.makedirs(d, exist_ok=True)
        dcp_io.save(module, optimizer, d, async_save=self.async_save)
        rank = dist.get_rank() if dist.is_initialized() else 0
        if rank == 0:
            extra = extra_state.__dict__ if isinstance(extra_state, ExtraState) else (extra_state or {})
            torch.save(extra, os.path.join(d, "extra_state.pth"))
        self._pending = (iteration, output_dir)

    def finish(self) -> None:
        dcp_io.wait()
        if self._pending is None:
            return
        iteration, output_dir = self._pending
        self._pending = None
        if dist.is_initialized():
            dist.barrier()
        if (dist.get_rank() if dist.is_initialized() else 0) == 0:
            tmp = os.path.join(output_dir, A.TRACKER_FILE + ".tmp")
            with open(tmp, "w") as f:
                f.write(str(iteration))
            os.replace(tmp, os.path.join(output_dir, A.TRACKER_FILE))


class FsdpShardDcpCkptLoader:
    def load(self, resume_from_ckpt: str, model=None, optimizer=None, extra_state: Optional[ExtraState] = None,
             ckpt_step: Optional[int] = None, **_):
        step = ckpt_step if ckpt_step is not None else A.latest_checkpoint_step(resume_from_ckpt)
        if dist.is_initialized():
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else "cpu"
            t = torch.tensor([-1 if step is None else step], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            step = int(t.item()) if t.item() >= 0 else None
        if step is None:
            return None
        d = os.path.join(resume_from_ckpt, f"iter_{step:07d}")
        if os.path.exists(os.path.join(d, ".metadata")):
            dcp_io.load(model, optimizer, d)
        else:
            A.load_checkpoint(model, optimizer, resume_from_ckpt, step)
        f = os.path.join(d, "extra_state.pth")
        if os.path.exists(f):
            st = torch.load(f, weights_only=False)
            if isinstance(extra_state, ExtraState):
                extra_state.__dict__.update(st)
            return st
        return {"iteration": step}
