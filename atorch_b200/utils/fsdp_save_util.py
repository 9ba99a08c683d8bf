"""Flat-parameter sharded checkpoints (the ATorch format) for the sharded engine.

Directory layout (RRRRR / WWWWW = zero-padded rank / world size of the shard group):

    ckpt_meta               pickle {"version": 1, "world_size": W, "wrap_class": {(module, class), ...}}
    buffers                 safetensors of model.named_buffers()                       (rank 0)
    flat_param.RRRRR-WWWWW  safetensors: unit name ("" = root) -> this rank's 1-D fp32 flat shard
    flat_meta.RRRRR-WWWWW   pickle {"flat_param_meta": {unit: {numels, flat_numel, numels_with_padding,
                            is_padding_mask}}, "param_meta": {fqn: {param_names, param_shapes,
                            param_numels, param_offsets=(start, end) inside the shard, pad, rank,
                            striped_fsdp_name}}}
    optim_param.RRRRR-WWWWW safetensors: "{fqn}-{state}" -> 1-D shard of that state (or scalar step)
    optim_meta              pickle: param_groups with "params" (fqn list) and "params_names"

A parameter's pieces on successive ranks are consecutive slices of the flattened parameter, so a
loader at ANY world size rebuilds what it needs from ``param_meta`` alone: it computes which pieces
overlap its own range and reads just those bytes (``SafeFile.get_slice``) - no rank-0 load, no
broadcast. ``ShardTensorUtil`` gives by-name access, ``load_fsdp_flat_param`` / ``ShardOptim`` fill
an engine and its optimizer at the current world size, ``ConvertFlatParam`` produces a full state
dict.
(Reference: atorch/utils/fsdp_save_util.py:139-1210.)
"""
from __future__ import annotations

import glob
import os
import pickle
from collections import defaultdict
from pathlib import Path
from typing import Callable, Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from .safetensors_io import SafeFile, save_file

CKPT_VERSION = 1


def _engine_of(model):
    eng = getattr(model, "engine", None)
    if eng is None:
        raise ValueError("model is not wrapped by the sharded engine (use the fsdp / zero optimisations)")
    return eng


def _suffix(rank: int, world: int) -> str:
    return f"{str(rank).zfill(5)}-{str(world).zfill(5)}"


def _unit_metas(eng) -> Tuple[Dict, Dict, Dict]:
    params, flat_meta, param_meta = {}, {}, {}
    for u in eng.units:
        shard = eng.master[u.shard_offset: u.shard_offset + u.shard_numel]
        params[u.name] = shard
        numels_wp, is_pad = [], []
        pos = 0
        for off, n in zip(u.offsets, u.numels):
            if off > pos:
                numels_wp.append(off - pos)
                is_pad.append(True)
            numels_wp.append(n)
            is_pad.append(False)
            pos = off + n
        if u.padded_numel > pos:
            numels_wp.append(u.padded_numel - pos)
            is_pad.append(True)
        flat_meta[u.name] = {"numels": tuple(u.numels), "flat_numel": u.shard_numel,
                             "numels_with_padding": tuple(numels_wp), "is_padding_mask": tuple(is_pad)}
        for fqn, shape, numel, (s, n, _) in zip(u.param_names, u.shapes, u.numels, u.param_shard_slices()):
            if n == 0:
                continue
            local = fqn[len(u.name) + 1:] if (u.name and fqn.startswith(u.name + ".")) else fqn
            param_meta[fqn] = {"param_names": local, "param_shapes": torch.Size(shape), "param_numels": numel,
                               "param_offsets": (s, s + n), "pad": u.padded_numel - u.numel, "rank": eng.rank,
                               "striped_fsdp_name": u.name}
    return params, flat_meta, param_meta


def save_fsdp_flat_param(model, path: str) -> None:
    """Every rank writes its flat shards and metadata; rank 0 also writes buffers and ``ckpt_meta``."""
    eng = _engine_of(model)
    Path(path).mkdir(parents=True, exist_ok=True)
    params, flat_meta, param_meta = _unit_metas(eng)
    suf = _suffix(eng.rank, eng.world)
    save_file({k: v.detach().cpu() for k, v in params.items()}, f"{path}/flat_param.{suf}")
    with open(f"{path}/flat_meta.{suf}", "wb") as f:
        pickle.dump({"flat_param_meta": flat_meta, "param_meta": param_meta}, f)
    if eng.rank == 0:
        save_file({n: b.detach().cpu() for n, b in eng.module.named_buffers()}, f"{path}/buffers")
    global_rank = dist.get_rank() if dist.is_initialized() else 0
    if global_rank == 0:
        wrap = {(type(u.module).__module__, type(u.module).__name__) for u in eng.units if not u.is_root}
        with open(f"{path}/ckpt_meta", "wb") as f:
            pickle.dump({"version": CKPT_VERSION, "world_size": eng.world, "wrap_class": wrap}, f)
    if dist.is_initialized():
        dist.barrier()


def _optimizer_state_by_fqn(eng, optimizer) -> Tuple[Dict[str, torch.Tensor], list]:
    """{"fqn-state": shard tensor} plus param_groups metadata for either optimizer flavour."""
    from ..parallel.fsdp import FusedShardedOptimizer

    out: Dict[str, torch.Tensor] = {}
    names = [n for n, _ in eng.shard_parameters()]
    if isinstance(optimizer, FusedShardedOptimizer):
        optimizer._ensure_state()
        for u in eng.units:
            for fqn, (s, n, _) in zip(u.param_names, u.param_shard_slices()):
                if n == 0:
                    continue
                lo = u.shard_offset + s
                out[f"{fqn}-exp_avg"] = optimizer.exp_avg[lo: lo + n]
                out[f"{fqn}-exp_avg_sq"] = optimizer.exp_avg_sq[lo: lo + n]
                out[f"{fqn}-step"] = torch.tensor(float(optimizer.step_count))
        groups = [dict({k: v for k, v in g.items() if k != "params"}, params=list(names),
                       params_names=dict(enumerate(names))) for g in optimizer.param_groups]
        return out, groups
    inner = getattr(optimizer, "optimizer", optimizer)
    by_id = {id(p): n for n, p in eng.shard_parameters()}
    for p, st in inner.state.items():
        fqn = by_id.get(id(p))
        if fqn is None or p.numel() == 0:
            continue
        for k, v in st.items():
            if isinstance(v, torch.Tensor):
                out[f"{fqn}-{k}"] = v.detach().reshape(-1) if v.dim() else v.detach()
    groups = []
    for g in inner.param_groups:
        gn = [by_id[id(p)] for p in g["params"] if id(p) in by_id]
        groups.append(dict({k: v for k, v in g.items() if k != "params"}, params=gn,
                           params_names=dict(enumerate(gn))))
    return out, groups


def save_fsdp_optim_param(model, optimizer, path: str) -> None:
    eng = _engine_of(model)
    Path(path).mkdir(parents=True, exist_ok=True)
    state, groups = _optimizer_state_by_fqn(eng, optimizer)
    save_file({k: v.detach().cpu() for k, v in state.items()}, f"{path}/optim_param.{_suffix(eng.rank, eng.world)}")
    if eng.rank == 0:
        with open(f"{path}/optim_meta", "wb") as f:
            pickle.dump(groups, f)
    if dist.is_initialized():
        dist.barrier()


class ShardTensorUtil:
    """By-name access to a flat checkpoint written at any world size.

    ``name_mapping_func_or_dict`` maps a requested name to the name stored in the checkpoint.
    """

    def __init__(self, path: str, rank: int = 0, world_size: int = 1, device="cpu",
                 name_mapping_func_or_dict: Union[None, Callable, Dict[str, str]] = None, create_param_cb=None,
                 prefix: str = "flat"):
        self.path, self.rank, self.world_size, self.device = path, rank, world_size, device
        self.name_mapping = name_mapping_func_or_dict
        self.create_param_cb = create_param_cb
        with open(f"{path}/ckpt_meta", "rb") as f:
            self.ckpt_meta = pickle.load(f)
        self.saved_world = self.ckpt_meta["world_size"]
        self.metas, self.files = [], []
        for r in range(self.saved_world):
            suf = _suffix(r, self.saved_world)
            with open(f"{path}/flat_meta.{suf}", "rb") as f:
                self.metas.append(pickle.load(f))
            self.files.append(SafeFile(f"{path}/flat_param.{suf}"))
        # fqn -> [(rank, unit, start_in_shard, end_in_shard)] in rank order, plus shape
        self.pieces: Dict[str, List[Tuple[int, str, int, int]]] = defaultdict(list)
        self.shapes: Dict[str, torch.Size] = {}
        for r, m in enumerate(self.metas):
            for fqn, pm in m["param_meta"].items():
                s, e = pm["param_offsets"]
                self.pieces[fqn].append((r, pm["striped_fsdp_name"], s, e))
                self.shapes[fqn] = torch.Size(pm["param_shapes"])
        self._buffers: Optional[SafeFile] = None

    def _map(self, name: str) -> str:
        if self.name_mapping is None:
            return name
        if callable(self.name_mapping):
            return self.name_mapping(name)
        return self.name_mapping.get(name, name)

    def param_names(self) -> List[str]:
        return list(self.pieces.keys())

    def load_param_slice(self, name: str, start: int, end: int) -> torch.Tensor:
        """Elements [start, end) of flattened parameter ``name`` (reads only overlapping pieces)."""
        fqn = self._map(name)
        if fqn not in self.pieces:
            raise KeyError(name)
        out, pos = [], 0
        for r, unit, s, e in self.pieces[fqn]:
            n = e - s
            lo, hi = max(start, pos), min(end, pos + n)
            if hi > lo:
                out.append(self.files[r].get_slice(unit, s + (lo - pos), s + (hi - pos)))
            pos += n
        return torch.cat(out) if out else torch.empty(0)

    def load_tensor_by_name(self, name: str, strict: bool = True) -> Optional[torch.Tensor]:
        fqn = self._map(name)
        if fqn in self.pieces:
            shape = self.shapes[fqn]
            return self.load_param_slice(name, 0, shape.numel()).view(shape).to(self.device)
        if self._buffers is None and os.path.exists(f"{self.path}/buffers"):
            self._buffers = SafeFile(f"{self.path}/buffers")
        if self._buffers is not None and fqn in self._buffers.header:
            return self._buffers.get_tensor(fqn).to(self.device)
        if strict:
            raise KeyError(name)
        return None

    def get_fsdp_init_order(self) -> List[str]:
        return list(self.metas[0]["flat_param_meta"].keys())

    def load_flat_param_by_name(self, unit_name: str, unit=None) -> torch.Tensor:
        """This rank's flat shard of ``unit`` (a ``FlatUnit`` of the current engine) rebuilt from the
        checkpoint, whatever world size it was written at."""
        assert unit is not None, "pass the FlatUnit to fill"
        out = torch.zeros(unit.shard_numel, dtype=torch.float32)
        for fqn, (s, n, ps) in zip(unit.param_names, unit.param_shard_slices()):
            if n:
                out[s: s + n] = self.load_param_slice(fqn, ps, ps + n).float()
        return out


def load_fsdp_flat_param(model, path: str, name_mapping=None) -> None:
    """Fill the engine's master shards (and buffers) from a flat checkpoint at the current world size."""
    eng = _engine_of(model)
    util = ShardTensorUtil(path, eng.rank, eng.world, "cpu", name_mapping)
    for u in eng.units:
        shard = util.load_flat_param_by_name(u.name, u)
        eng.master[u.shard_offset: u.shard_offset + u.shard_numel].copy_(shard)
    eng.sync_working_copy()
    for n, b in eng.module.named_buffers():
        t = util.load_tensor_by_name(n, strict=False)
        if t is not None:
            b.copy_(t)


class ShardOptim:
    """Optimizer state of a flat checkpoint, resliced to the current sharding."""

    def __init__(self, path: str):
        self.path = path
        with open(f"{path}/optim_meta", "rb") as f:
            self.param_groups = pickle.load(f)
        files = sorted(glob.glob(f"{path}/optim_param.*"))
        self.saved_world = len(files)
        self.files = [SafeFile(f"{path}/optim_param.{_suffix(r, self.saved_world)}") for r in range(self.saved_world)]
        self.state_names = set()
        self.pieces: Dict[str, List[Tuple[int, int]]] = defaultdict(list)   # key -> [(rank, numel)]
        for r, f in enumerate(self.files):
            for k in f.keys():
                _, shape = f.info(k)
                n = 1
                for s in shape:
                    n *= s
                self.pieces[k].append((r, n if shape else 0))
                self.state_names.add(k.rsplit("-", 1)[1])

    def load_state_slice(self, fqn: str, state: str, start: int, end: int) -> Optional[torch.Tensor]:
        key = f"{fqn}-{state}"
        if key not in self.pieces:
            return None
        out, pos = [], 0
        for r, n in self.pieces[key]:
            if n == 0:       # scalar (e.g. step): same on every rank
                return self.files[r].get_tensor(key)
            lo, hi = max(start, pos), min(end, pos + n)
            if hi > lo:
                out.append(self.files[r].get_slice(key, lo - pos, hi - pos))
            pos += n
        return torch.cat(out) if out else torch.empty(0)

    def reshard_optim_state_dict(self, model) -> Dict:
        """``{"state": {fqn: {state: shard tensor}}, "param_groups": [...]}`` for this rank."""
        eng = _engine_of(model)
        state: Dict[str, Dict[str, torch.Tensor]] = {}
        for u in eng.units:
            for fqn, (s, n, ps) in zip(u.param_names, u.param_shard_slices()):
                if n == 0:
                    continue
                st = {}
                for name in self.state_names:
                    t = self.load_state_slice(fqn, name, ps, ps + n)
                    if t is not None:
                        st[name] = t
                state[fqn] = st
        return {"state": state, "param_groups": self.param_groups}

    def load_into(self, model, optimizer) -> None:
        from ..parallel.fsdp import FusedShardedOptimizer

        eng = _engine_of(model)
        sd = self.reshard_optim_state_dict(model)
        if isinstance(optimizer, FusedShardedOptimizer):
            optimizer._ensure_state()
            for u in eng.units:
                for fqn, (s, n, _) in zip(u.param_names, u.param_shard_slices()):
                    if n == 0 or fqn not in sd["state"]:
                        continue
                    lo = u.shard_offset + s
                    st = sd["state"][fqn]
                    optimizer.exp_avg[lo: lo + n].copy_(st["exp_avg"])
                    optimizer.exp_avg_sq[lo: lo + n].copy_(st["exp_avg_sq"])
                    if "step" in st:
                        optimizer.step_count = int(st["step"].item())
            for g, saved in zip(optimizer.param_groups, sd["param_groups"]):
                g.update({k: v for k, v in saved.items() if k not in ("params", "params_names")})
            return
        inner = getattr(optimizer, "optimizer", optimizer)
        for name, p in eng.shard_parameters():
            if p.numel() == 0 or name not in sd["state"]:
                continue
            st = {k: (v.view_as(p).to(p.device) if v.numel() == p.numel() and v.dim() else v.to(p.device))
                  for k, v in sd["state"][name].items()}
            inner.state[p] = st


class ConvertFlatParam:
    """Whole-model state dict out of a flat checkpoint (no distributed job needed)."""

    def __init__(self, path: str):
        self.util = ShardTensorUtil(path)

    def convert(self) -> Dict[str, torch.Tensor]:
        sd = {n: self.util.load_tensor_by_name(n) for n in self.util.param_names()}
        if os.path.exists(f"{self.util.path}/buffers"):
            bf = SafeFile(f"{self.util.path}/buffers")
            for k in bf.keys():
                sd[k] = bf.get_tensor(k)
        return sd
