"""Asynchronous flat checkpoints: ``save_checkpoint(step, model, optimizer, path, ...)`` copies this
rank's shards to pinned host memory (the only part the training loop waits for) and a writer thread
persists them in the flat format of :mod:`fsdp_save_util`; the tracker file
``latest_checkpointed_iteration.txt`` is updated only after every rank's files are complete.
``storage_type=MEMORY`` keeps the host copy without writing (fast in-memory restore after a restart
of the training loop inside the same process).
(Reference: atorch/utils/fsdp_async_ckpt_util.py:29-216, which hands the shared-memory copy to the
dlrover flash-checkpoint agent.)
"""
from __future__ import annotations

import os
import pickle
import threading
from enum import Enum
from pathlib import Path
from typing import Dict, Optional

import torch
import torch.distributed as dist

from .fsdp_save_util import CKPT_VERSION, _engine_of, _optimizer_state_by_fqn, _suffix, _unit_metas
from .safetensors_io import save_file

TRACKER_FILE = "latest_checkpointed_iteration.txt"


class StorageType(Enum):
    MEMORY = "memory"
    DISK = "disk"


class _Writer:
    def __init__(self):
        self.thread: Optional[threading.Thread] = None
        self.error: Optional[BaseException] = None
        self.memory: Dict[int, dict] = {}

    def wait(self) -> None:
        if self.thread is not None:
            self.thread.join()
            self.thread = None
        if self.error is not None:
            e, self.error = self.error, None
            raise e


_WRITER = _Writer()


def _to_pinned(t: torch.Tensor) -> torch.Tensor:
    if not t.is_cuda:
        return t.detach().clone()
    host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
    host.copy_(t, non_blocking=True)
    return host


def save_checkpoint(step: int, model, optimizer, path: str, extra_sds: Optional[dict] = None,
                    extra_paths: Optional[dict] = None, storage_type: StorageType = StorageType.DISK,
                    block: bool = False) -> None:
    eng = _engine_of(model)
    _WRITER.wait()                              # one checkpoint in flight at a time
    params, flat_meta, param_meta = _unit_metas(eng)
    host_params = {k: _to_pinned(v) for k, v in params.items()}
    opt_state, groups = _optimizer_state_by_fqn(eng, optimizer) if optimizer is not None else ({}, [])
    host_opt = {k: _to_pinned(v) for k, v in opt_state.items()}
    buffers = {n: _to_pinned(b) for n, b in eng.module.named_buffers()} if eng.rank == 0 else {}
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()
    payload = dict(step=step, params=host_params, metas={"flat_param_meta": flat_meta, "param_meta": param_meta},
                   opt=host_opt, groups=groups, buffers=buffers, extra=extra_sds or {})
    if storage_type == StorageType.MEMORY:
        _WRITER.memory = {step: payload}
        return
    out = os.path.join(path, f"iter_{step:07d}") if not path.endswith(f"{step}") else path
    rank, world = eng.rank, eng.world
    wrap = {(type(u.module).__module__, type(u.module).__name__) for u in eng.units if not u.is_root}
    global_rank = dist.get_rank() if dist.is_initialized() else 0

    def write():
        try:
            Path(out).mkdir(parents=True, exist_ok=True)
            suf = _suffix(rank, world)
            save_file(payload["params"], f"{out}/flat_param.{suf}")
            with open(f"{out}/flat_meta.{suf}", "wb") as f:
                pickle.dump(payload["metas"], f)
            if payload["opt"]:
                save_file(payload["opt"], f"{out}/optim_param.{suf}")
            if rank == 0:
                save_file(payload["buffers"], f"{out}/buffers")
                with open(f"{out}/optim_meta", "wb") as f:
                    pickle.dump(payload["groups"], f)
            if global_rank == 0:
                with open(f"{out}/ckpt_meta", "wb") as f:
                    pickle.dump({"version": CKPT_VERSION, "world_size": world, "wrap_class": wrap}, f)
            for name, sd in payload["extra"].items():
                if global_rank == 0:
                    torch.save(sd, (extra_paths or {}).get(name, f"{out}/{name}.pt"))
            with open(f"{out}/.done.{suf}", "w") as f:
                f.write("ok")
            if global_rank == 0:
                # the tracker moves only when every rank has finished its files
                import time

                t0 = time.time()
                while not all(os.path.exists(f"{out}/.done.{_suffix(r, world)}") for r in range(world)):
                    if time.time() - t0 > 600:
                        raise TimeoutError("other ranks did not finish their checkpoint files")
                    time.sleep(0.05)
                tmp = os.path.join(path, TRACKER_FILE + ".tmp")
                with open(tmp, "w") as f:
                    f.write(str(step))
                os.replace(tmp, os.path.join(path, TRACKER_FILE))
        except BaseException as e:   # surfaced at the next wait()
            _WRITER.error = e
    _WRITER.thread = threading.Thread(target=write, daemon=True)
    _WRITER.thread.start()
    if block:
        _WRITER.wait()


def wait_for_checkpoint() -> None:
    _WRITER.wait()


def latest_checkpoint_step(path: str) -> Optional[int]:
    f = os.path.join(path, TRACKER_FILE)
    if not os.path.exists(f):
        return None
    with open(f) as fh:
        return int(fh.read().strip())


def load_checkpoint(model, optimizer, path: str, step: Optional[int] = None) -> Optional[int]:
    """Load the checkpoint named by the tracker file (or ``step``); returns the step or None."""
    from .fsdp_save_util import ShardOptim, load_fsdp_flat_param

    step = step if step is not None else latest_checkpoint_step(path)
    if step is None:
        return None
    d = os.path.join(path, f"iter_{step:07d}")
    load_fsdp_flat_param(model, d)
    if optimizer is not None and os.path.exists(os.path.join(d, "optim_meta")):
        ShardOptim(d).load_into(model, optimizer)
    return step
