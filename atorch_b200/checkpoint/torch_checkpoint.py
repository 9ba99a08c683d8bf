"""``TorchDCPCheckpointManager``: step-numbered sharded checkpoints ``{folder}/step-{n}/`` holding model,
optimizer, lr scheduler, dataloader and train state, written with ``torch.distributed.checkpoint``
for plain / DDP models and with the flat shard format for the sharded engine; ``keep_latest_k`` rotation.
(Reference: atorch/checkpoint/torch_checkpoint.py:38-170.)"""
from __future__ import annotations

import os
import re
import shutil
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist


class TorchDCPCheckpointManager:
    def __init__(self, save_load_folder: str, interval: int = 1, keep_latest_k: int = 0, async_mode: bool = False):
        self.folder, self.interval, self.keep_latest_k, self.async_mode = save_load_folder, interval, keep_latest_k, async_mode
        os.makedirs(save_load_folder, exist_ok=True)

    def _dir(self, step: int) -> str:
        return os.path.join(self.folder, f"step-{step}")

    def steps(self):
        pat = re.compile(r"^step-(\d+)$")
        return sorted(int(m.group(1)) for d in os.listdir(self.folder) if (m := pat.match(d)))

    def save(self, curr_step: int, model, optimizer=None, lr_scheduler=None, dataloader=None,
             train_state: Optional[Dict[str, Any]] = None, force: bool = False) -> bool:
        if not force and curr_step % self.interval != 0:
            return False
        d = self._dir(curr_step)
        rank = dist.get_rank() if dist.is_initialized() else 0
        if hasattr(model, "engine"):
            from ..utils.fsdp_save_util import save_fsdp_flat_param, save_fsdp_optim_param

            save_fsdp_flat_param(model, d)
            if optimizer is not None:
                save_fsdp_optim_param(model, optimizer, d)
        else:
            import torch.distributed.checkpoint as dcp

            state = {"model": model.state_dict()}
            if optimizer is not None:
                state["optim"] = optimizer.state_dict()
            if dist.is_initialized():
                dcp.save(state, checkpoint_id=d)
            elif rank == 0:
                os.makedirs(d, exist_ok=True)
                torch.save(state, os.path.join(d, "state.pt"))
        if rank == 0:
            os.makedirs(d, exist_ok=True)
            extra = {"train_state": train_state or {}}
            if lr_scheduler is not None:
                extra["lr_scheduler"] = lr_scheduler.state_dict()
            if dataloader is not None and hasattr(dataloader, "state_dict"):
                extra["dataloader"] = dataloader.state_dict()
            torch.save(extra, os.path.join(d, "extra_state.pt"))
            if self.keep_latest_k > 0:
                for s in self.steps()[:-self.keep_latest_k]:
                    shutil.rmtree(self._dir(s), ignore_errors=True)
        if dist.is_initialized():
            dist.barrier()
        return True

    def load(self, model, optimizer=None, lr_scheduler=None, dataloader=None, step: int = -1) -> Optional[Dict]:
        steps = self.steps()
        if not steps:
            return None
        step = steps[-1] if step < 0 else step
        d = self._dir(step)
        if hasattr(model, "engine"):
            from ..utils.fsdp_save_util import ShardOptim, load_fsdp_flat_param

            load_fsdp_flat_param(model, d)
            if optimizer is not None and os.path.exists(os.path.join(d, "optim_meta")):
                ShardOptim(d).load_into(model, optimizer)
        elif os.path.exists(os.path.join(d, "state.pt")):
            st = torch.load(os.path.join(d, "state.pt"), map_location="cpu")
            model.load_state_dict(st["model"])
            if optimizer is not None and "optim" in st:
                optimizer.load_state_dict(st["optim"])
        else:
            import torch.distributed.checkpoint as dcp

            state = {"model": model.state_dict()}
            if optimizer is not None:
                state["optim"] = optimizer.state_dict()
            dcp.load(state, checkpoint_id=d)
            model.load_state_dict(state["model"])
            if optimizer is not None:
                optimizer.load_state_dict(state["optim"])
        extra = torch.load(os.path.join(d, "extra_state.pt"), weights_only=False)
        if lr_scheduler is not None and "lr_scheduler" in extra:
            lr_scheduler.load_state_dict(extra["lr_scheduler"])
        if dataloader is not None and "dataloader" in extra and hasattr(dataloader, "load_state_dict"):
            dataloader.load_state_dict(extra["dataloader"])
        return dict(extra.get("train_state", {}), step=step)
