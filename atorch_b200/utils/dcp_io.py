"""Sharded checkpoints of the sharded engine in the ``torch.distributed.checkpoint`` (DCP) file format:
``.metadata`` plus one ``__{rank}_{n}.distcp`` file per rank, under the state key ``"atorch_FsdpShardDcpCkpt"``
→ ``{"model": ..., "optim": ...}``.

Every parameter is saved under its fully qualified name as a 1-D tensor of its ``numel``; a rank contributes
the slice ``[start, end)`` that lies in its flat shard (an uneven ``ShardedTensor`` built from local shards;
ranks that hold nothing of a parameter contribute no shard). Optimizer states use ``"{fqn}-{state}"`` with
the same slicing; scalar states (``step``) are plain tensors. Because the file describes parameters, not
flat units, it loads at any world size and any unit alignment: the loader builds the same structure over
the current shards — whose tensors are *views of the engine's buffers* — and DCP fills them in place.

Without an initialised process group the tensors are saved whole (DCP's single-process mode).
(Reference: atorch/trainer/fsdp/fsdp_shard_async_saver.py:77-131, dcp_forked.py:25-186,
fsdp_shard_dcp_loader.py:19-91.)
"""
from __future__ import annotations

import threading
from typing import Dict, Optional

import torch
import torch.distributed as dist

STATE_KEY = "atorch_FsdpShardDcpCkpt"


def _engine_of(model):
    eng = getattr(model, "engine", None)
    if eng is None:
        raise ValueError("model is not wrapped by the sharded engine (use the fsdp / zero optimisations)")
    return eng


def _placement(rank: int, t: torch.Tensor) -> str:
    return f"rank:{rank}/{'cuda:%d' % t.device.index if t.is_cuda else 'cpu'}"


def _wrap(local: Optional[torch.Tensor], start: int, numel: int, group, stage: bool):
    """1-D tensor of ``numel`` elements of which this rank holds ``local`` at offset ``start``."""
    if not dist.is_initialized():
        return local
    from torch.distributed._shard.sharded_tensor import Shard, ShardedTensor, ShardMetadata

    shards = []
    if local is not None and local.numel() > 0:
        t = local.detach().cpu().clone() if stage else local.detach()
        shards.append(Shard(t, ShardMetadata(shard_offsets=[start], shard_sizes=[t.numel()],
                                             placement=_placement(dist.get_rank(), t))))
    return ShardedTensor._init_from_local_shards(shards, [numel], process_group=group)


def engine_state(model, optimizer=None, stage: bool = False, group=None) -> Dict[str, Dict]:
    """``{"model": {fqn: tensor}, "optim": {"{fqn}-{state}": tensor}}`` over this rank's shards. With
    ``stage`` the local pieces are host copies (for a background writer); otherwise they are views of the
    engine's master / optimizer-state buffers, which is what loading needs."""
    from ..parallel.fsdp import FusedShardedOptimizer

    eng = _engine_of(model)
    out: Dict[str, Dict] = {"model": {}, "optim": {}}
    fused = isinstance(optimizer, FusedShardedOptimizer)
    if fused:
        optimizer._ensure_state()
    inner = getattr(optimizer, "optimizer", optimizer) if optimizer is not None and not fused else None
    shard_params = dict(eng.shard_parameters()) if inner is not None else {}
    # wrapping a tensor is a collective (shard metadata is exchanged), so every rank must wrap the same
    # keys in the same order, whether or not it holds a piece: agree on the optimizer's tensor state names
    state_names = []
    if inner is not None:
        mine = sorted({k for st in inner.state.values() for k, v in st.items()
                       if isinstance(v, torch.Tensor) and v.dim() > 0})
        if dist.is_initialized():
            lists = [None] * dist.get_world_size(group)
            dist.all_gather_object(lists, mine, group=group)
            mine = sorted({k for l in lists for k in l})
        state_names = mine
    for u in eng.units:
        for fqn, numel, (s, n, off) in zip(u.param_names, u.numels, u.param_shard_slices()):
            lo = u.shard_offset + s
            piece = eng.master[lo: lo + n] if n > 0 else None
            out["model"][fqn] = _wrap(piece, off, numel, group, stage) if dist.is_initialized() else \
                _whole(piece, numel, stage)
            if fused:
                for name, buf in (("exp_avg", optimizer.exp_avg), ("exp_avg_sq", optimizer.exp_avg_sq)):
                    sp = buf[lo: lo + n] if n > 0 else None
                    out["optim"][f"{fqn}-{name}"] = _wrap(sp, off, numel, group, stage) if dist.is_initialized() \
                        else _whole(sp, numel, stage)
            elif inner is not None:
                p = shard_params.get(fqn)
                st = inner.state.get(p, {}) if p is not None else {}
                for name in state_names:
                    v = st.get(name)
                    sp = v.detach().reshape(-1) if (isinstance(v, torch.Tensor) and n > 0 and v.numel() == n) else None
                    if dist.is_initialized():
                        out["optim"][f"{fqn}-{name}"] = _wrap(sp, off, numel, group, stage)
                    elif sp is not None:
                        out["optim"][f"{fqn}-{name}"] = _whole(sp, numel, stage)
    if fused:
        out["optim"]["step"] = torch.tensor(float(optimizer.step_count))
    elif inner is not None:
        steps = [float(st["step"]) for st in inner.state.values() if "step" in st]
        out["optim"]["step"] = torch.tensor(max(steps) if steps else 0.0)
    for name, b in eng.module.named_buffers():
        out["model"][f"buffer.{name}"] = b.detach().cpu().clone() if stage else b.detach()
    return out


def _whole(piece: Optional[torch.Tensor], numel: int, stage: bool):
    assert piece is not None and piece.numel() == numel, "a single process holds every parameter whole"
    return piece.detach().cpu().clone() if stage else piece.detach()


class _Pending:
    def __init__(self):
        self.thread: Optional[threading.Thread] = None
        self.error: Optional[BaseException] = None

    def wait(self) -> None:
        if self.thread is not None:
            self.thread.join()
            self.thread = None
        if self.error is not None:
            e, self.error = self.error, None
            raise e


_PENDING = _Pending()
def _io_group(eng):
    """``(gloo group over the ranks that share this engine's shards, writes?)``. The checkpoint holds each
    element once: with replicated shard groups (hybrid sharding) only the replica that contains global
    rank 0 writes, every replica reads. The default group may be NCCL-only, and a background writer must
    not share a communicator with training collectives, hence a gloo group of its own (cached per engine)."""
    if not dist.is_initialized():
        return None, True
    cached = getattr(eng, "_dcp_io_group", None)
    if cached is not None:
        return cached
    mine = dist.get_process_group_ranks(eng.group if eng.group is not None else dist.group.WORLD) \
        if eng.world > 1 else [dist.get_rank()]
    lists = [None] * dist.get_world_size()
    dist.all_gather_object(lists, sorted(mine))
    group = None
    for ranks in sorted({tuple(x) for x in lists}):
        g = dist.new_group(ranks=list(ranks), backend="gloo")     # collective: every rank creates every group
        if dist.get_rank() in ranks:
            group = g
    eng._dcp_io_group = (group, 0 in mine)
    return eng._dcp_io_group


def save(model, optimizer, path: str, async_save: bool = False) -> None:
    """Write a DCP checkpoint into ``path``. ``async_save``: the shards are copied to host memory first and
    a background thread writes them; ``wait()`` joins it (and re-raises its error)."""
    import torch.distributed.checkpoint as dcp

    _PENDING.wait()
    group, writes = _io_group(_engine_of(model))
    if not writes:
        return
    state = {STATE_KEY: engine_state(model, optimizer, stage=True, group=group)}
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()

    def write():
        try:
            dcp.save(state, checkpoint_id=path, process_group=group)
        except BaseException as e:  # noqa: BLE001 - surfaced at wait()
            _PENDING.error = e
    if async_save:
        _PENDING.thread = threading.Thread(target=write, daemon=True)
        _PENDING.thread.start()
    else:
        write()
        _PENDING.wait()


def wait() -> None:
    _PENDING.wait()


def load(model, optimizer, path: str) -> None:
    """Fill the engine's master shards, optimizer state and buffers from a DCP checkpoint written at any
    world size, then refresh the working copies."""
    import torch.distributed.checkpoint as dcp

    from ..parallel.fsdp import FusedShardedOptimizer

    _PENDING.wait()
    eng = _engine_of(model)
    group, _ = _io_group(eng)
    on_gpu = eng.master.is_cuda
    st = engine_state(model, optimizer, stage=on_gpu, group=group)     # host staging when the buffers are on a GPU
    want_step = "step" in st["optim"]
    dcp.load({STATE_KEY: st}, checkpoint_id=path, process_group=group)
    if on_gpu:   # copy the staged pieces back into the device buffers
        live = engine_state(model, optimizer, stage=False, group=group)
        for part in ("model", "optim"):
            for k, v in st[part].items():
                dst = live[part].get(k)
                if dst is None:
                    continue
                if hasattr(v, "local_shards"):
                    for a, b in zip(dst.local_shards(), v.local_shards()):
                        a.tensor.copy_(b.tensor)
                elif k != "step":
                    dst.copy_(v)
    if want_step and optimizer is not None:
        step = int(st["optim"]["step"].item())
        if isinstance(optimizer, FusedShardedOptimizer):
            optimizer.step_count = step
        else:
            inner = getattr(optimizer, "optimizer", optimizer)
            for s in inner.state.values():
                if "step" in s:
                    s["step"] = torch.tensor(float(step)) if isinstance(s["step"], torch.Tensor) else step
    eng.sync_working_copy()
