"""Process-group runtime: ``init_distributed`` and named parallel groups.

One process per GPU, ``torch.distributed`` (NCCL on GPUs, Gloo on CPUs) as the control plane.
Named groups are described by a *parallel config*
``([(name, size), ...], rank_order | None[, multi_instance[, use_device_mesh]])`` whose first name
varies fastest over the ranks: ``[("tensor", 4), ("pipeline", 2), ("data", 2)]`` on 16 ranks gives
tensor groups ``[0..3], [4..7], ...``, pipeline groups ``[0, 4], [1, 5], ...`` and data groups
``[0, 8], [1, 9], ...``. The rank sets are computed by plain mixed-radix arithmetic
(:func:`compute_group_ranks`), so they can be tested without any process group.

Same public behaviour as atorch/distributed/distributed.py:51-1026 of the reference
(``create_parallel_group`` :429-541, ``get_data_partition_rank_and_size`` :587-611,
sequence-parallel groups and ``seq_all_to_all`` :613-679, ``init_distributed`` :842-996).
"""
from __future__ import annotations

import datetime
import logging
import os
import socket
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

logger = logging.getLogger("atorch.logger")

SlicingDim = Sequence[Tuple[str, int]]
_SP_NAME = "sequence"


class _State:
    """All mutable process-level state of the runtime (one instance, reset by ``reset_distributed``)."""

    def __init__(self):
        self.initialized = False
        self.backend: Optional[str] = None
        self.rank: Optional[int] = None
        self.local_rank: Optional[int] = None
        self.world_size: Optional[int] = None
        self.nproc_per_node: Optional[int] = None
        self.node_size: Optional[int] = None
        self.coworker_size = 0
        self.prefix = ""
        # keyed by prefixed group name
        self.group: Dict[str, dist.ProcessGroup] = {}
        self.group_rank: Dict[str, int] = {}
        self.group_size: Dict[str, int] = {}
        self.groups_and_ranks: Dict[str, List[Tuple[Optional[dist.ProcessGroup], List[int]]]] = {}
        # keyed by prefix
        self.config: Dict[str, list] = {}
        self.instance_num: Dict[str, int] = {}
        self.instance_index: Dict[str, Optional[int]] = {}
        self.meshes: list = []
        self.owned_groups: List[dist.ProcessGroup] = []


_S = _State()


class ParallelGroupContextManager:
    """Within the context, group names are prefixed with ``name`` so several independent sets of
    parallel groups (e.g. actor / critic models of RLHF) can coexist."""

    def __init__(self, name: str = ""):
        self.name = name
        self._old = ""

    def __enter__(self):
        self._old = _S.prefix
        _S.prefix = self.name
        return self

    def __exit__(self, *exc):
        _S.prefix = self._old


def _pname(name: str = "") -> str:
    return _S.prefix + name


# --------------------------------------------------------------------------------------------
# basic queries
# --------------------------------------------------------------------------------------------
def rank() -> Optional[int]:
    if _S.rank is not None:
        return _S.rank
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else None


def local_rank() -> int:
    if _S.local_rank is not None:
        return _S.local_rank
    return 0 if not (dist.is_available() and dist.is_initialized()) else int(os.getenv("LOCAL_RANK", -1))


def world_size() -> Optional[int]:
    if _S.world_size:
        return _S.world_size
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else None


def nproc_per_node() -> Optional[int]:
    return _S.nproc_per_node


def node_size() -> Optional[int]:
    return _S.node_size


def coworker_size() -> int:
    return _S.coworker_size


def backend() -> Optional[str]:
    return _S.backend


def is_distributed() -> bool:
    ws = world_size()
    return ws is not None and ws > 1


def is_coworker() -> bool:
    return False


def parallel_group(name: str) -> Optional[dist.ProcessGroup]:
    return _S.group.get(_pname(name))


def parallel_rank(name: str) -> Optional[int]:
    return _S.group_rank.get(_pname(name))


def parallel_group_size(name: str) -> Optional[int]:
    return _S.group_size.get(_pname(name))


def parallel_config():
    return _S.config.get(_pname())


def parallel_instance_num() -> Optional[int]:
    return _S.instance_num.get(_pname())


def parallel_instance_index() -> Optional[int]:
    return _S.instance_index.get(_pname())


def parallel_group_and_ranks(name: str):
    """(group, ranks) of the group named ``name`` that contains this rank, or (None, None)."""
    entries = _S.groups_and_ranks.get(_pname(name))
    if entries is not None:
        me = rank()
        for g, ranks in entries:
            if me in ranks:
                return g, ranks
        return None, None
    g = parallel_group(name)
    return g, (list(range(world_size())) if g is not None else None)


def get_group_name(group) -> Optional[str]:
    for n, g in _S.group.items():
        if g is group:
            return n
    return None


def pipe_prev_rank() -> Optional[int]:
    r = parallel_rank("pipe")
    if r is None:
        return None
    _, ranks = parallel_group_and_ranks("pipe")
    return ranks[(r - 1) % len(ranks)]


def pipe_next_rank() -> Optional[int]:
    r = parallel_rank("pipe")
    if r is None:
        return None
    _, ranks = parallel_group_and_ranks("pipe")
    return ranks[(r + 1) % len(ranks)]


def is_pipe_first_stage(ignore_virtual: bool = True, true_if_no_pipe: bool = True) -> bool:
    r = parallel_rank("pipe")
    if r is None:
        return true_if_no_pipe
    return r == 0


def is_pipe_last_stage(ignore_virtual: bool = True, true_if_no_pipe: bool = True) -> bool:
    r = parallel_rank("pipe")
    if r is None:
        return true_if_no_pipe
    return r == parallel_group_size("pipe") - 1


# --------------------------------------------------------------------------------------------
# rank-set arithmetic (pure)
# --------------------------------------------------------------------------------------------
def compute_group_ranks(slicing_dim: SlicingDim, rank_order: Sequence[int], offset: int = 0) -> Dict[str, List[List[int]]]:
    """Rank sets of every named group of ONE parallel instance starting at ``rank_order[offset]``.

    Position ``p`` inside the instance decomposes as mixed-radix digits, first name least
    significant; the groups of a name are the sets of positions that differ only in that digit.
    """
    sizes = [s for _, s in slicing_dim]
    total = 1
    for s in sizes:
        total *= s
    out: Dict[str, List[List[int]]] = {}
    stride = 1
    for name, size in slicing_dim:
        groups = []
        for base in range(total):
            if (base // stride) % size != 0:
                continue
            groups.append([rank_order[offset + base + i * stride] for i in range(size)])
        out[name] = groups
        stride *= size
    return out


def get_pg_ranks(slicing_dim: SlicingDim, rank_order: Sequence[int], world: Optional[int] = None):
    """List (one entry per parallel instance) of ``{name: [ranks, ...]}``."""
    world = world if world is not None else world_size()
    total = 1
    for _, s in slicing_dim:
        total *= s
    return [compute_group_ranks(slicing_dim, rank_order, i * total) for i in range(world // total)]


def get_ranks_in_same_group(parallel_mode, my_rank: int = 0, world: Optional[int] = None) -> Dict[str, List[int]]:
    slicing_dim, order = parallel_mode[0], parallel_mode[1]
    world = world if world is not None else world_size()
    order = list(range(world)) if order is None else order
    res = {}
    for inst in get_pg_ranks(slicing_dim, order, world):
        for name, groups in inst.items():
            for ranks in groups:
                if my_rank in ranks:
                    res[name] = ranks
    return res


# --------------------------------------------------------------------------------------------
# group creation
# --------------------------------------------------------------------------------------------
def _register(name: str, size: int, ranks_list: List[List[int]], make_group=True):
    pn = _pname(name)
    if pn in _S.group_size:
        raise ValueError(f"group name {pn!r} already used")
    entries = []
    me = rank()
    for ranks in ranks_list:
        g = dist.new_group(ranks) if make_group else None
        if g is not None:
            _S.owned_groups.append(g)
        entries.append((g, list(ranks)))
        if me in ranks:
            _S.group[pn] = g
            _S.group_rank[pn] = list(ranks).index(me)
    _S.groups_and_ranks[pn] = entries
    _S.group_size[pn] = size


def build_mesh(slicing_dim: SlicingDim, prefix: str = "", reverse_order: bool = True):
    """``torch.distributed.DeviceMesh`` whose dims are the (prefixed) names; with ``reverse_order``
    the last name becomes the outermost mesh dim so that mesh groups equal the list-order groups."""
    from torch.distributed.device_mesh import init_device_mesh

    dims = list(slicing_dim)[::-1] if reverse_order else list(slicing_dim)
    device_type = "cuda" if (_S.backend or "").find("nccl") >= 0 and torch.cuda.is_available() else "cpu"
    return init_device_mesh(device_type, tuple(s for _, s in dims), mesh_dim_names=tuple(prefix + n for n, _ in dims))


def get_device_mesh(group_name: str, use_prefix: bool = True):
    pn = _pname(group_name) if use_prefix else group_name
    for mesh in _S.meshes:
        if pn in mesh.mesh_dim_names:
            return mesh[pn]
    return None


def get_root_device_mesh(group_name: str, use_prefix: bool = True):
    pn = _pname(group_name) if use_prefix else group_name
    for mesh in _S.meshes:
        if pn in mesh.mesh_dim_names:
            return mesh
    return None


def create_parallel_group(parallel_config, use_atorch_pipe: bool = True, use_device_mesh: bool = False,
                          reverse_mesh_pg_order: bool = True) -> None:
    """Create the named groups of ``parallel_config`` (see module docstring). A single dim covering
    the whole world reuses the default group instead of creating a new communicator."""
    assert _S.initialized or dist.is_initialized(), "distributed should be initialized"
    slicing_dim = [(n, int(s)) for n, s in parallel_config[0]]
    rank_order = parallel_config[1]
    multi = parallel_config[2] if len(parallel_config) > 2 else False
    use_device_mesh = use_device_mesh or (parallel_config[3] if len(parallel_config) > 3 else False)
    assert len(slicing_dim) > 0, "parallel_config should not be empty"
    total = 1
    for _, s in slicing_dim:
        total *= s
    ws = world_size()
    if not multi and ws != total:
        raise ValueError(f"product of parallel sizes ({total}) must equal world size ({ws}): {parallel_config}")
    if use_device_mesh and rank_order is not None:
        raise NotImplementedError("rank_order with device mesh")
    order = list(range(ws)) if rank_order is None else list(rank_order)
    _S.config[_pname()] = [slicing_dim, order, multi]
    n_inst = ws // total
    me = rank()
    _S.instance_num[_pname()] = n_inst
    _S.instance_index[_pname()] = me // total if me < n_inst * total else None

    if len(slicing_dim) == 1 and ws == total and not use_device_mesh:
        name, size = slicing_dim[0]
        pn = _pname(name)
        if pn in _S.group_size:
            raise ValueError(f"group name {pn!r} already used")
        _S.group[pn] = dist.group.WORLD
        _S.group_rank[pn] = me
        _S.group_size[pn] = size
    elif use_device_mesh:
        mesh = build_mesh(slicing_dim, _S.prefix, reverse_mesh_pg_order if len(slicing_dim) > 1 else False)
        _S.meshes.append(mesh)
        for name, size in slicing_dim:
            pn = _pname(name)
            g = mesh.get_group(pn)
            ranks = dist.get_process_group_ranks(g)
            _S.group[pn] = g
            _S.group_rank[pn] = ranks.index(me)
            _S.group_size[pn] = size
            _S.groups_and_ranks[pn] = [(g, ranks)]
    else:
        inst = get_pg_ranks(slicing_dim, order, ws)
        for name, size in slicing_dim:
            _register(name, size, [r for i in range(n_inst) for r in inst[i][name]])
    if any(n == "pipe" for n, _ in slicing_dim) and use_atorch_pipe and torch.cuda.is_available() \
            and (_S.backend or "").find("nccl") >= 0:
        # a first collective on the pipe communicator makes later batched isend/irecv safe
        t = torch.ones(1, device=torch.device("cuda", local_rank()))
        dist.all_reduce(t, group=parallel_group("pipe"))


def destroy_parallel_group(destroy_rpc: bool = True) -> None:
    for g in _S.owned_groups:
        try:
            dist.destroy_process_group(g)
        except Exception:  # already gone
            pass
    _S.owned_groups.clear()
    _S.group.clear()
    _S.group_rank.clear()
    _S.group_size.clear()
    _S.groups_and_ranks.clear()
    _S.config.clear()
    _S.instance_num.clear()
    _S.instance_index.clear()
    _S.meshes.clear()


def get_data_partition_rank_and_size() -> Tuple[int, int]:
    """(rank, size) of the data partition = ``data`` x ``zero`` groups divided by sequence parallel."""
    dsize, drank = parallel_group_size("data"), parallel_rank("data")
    if dsize is None:
        dsize, drank = 1, 0
    zsize = parallel_group_size("zero")
    if zsize is not None:
        drank = drank * zsize + parallel_rank("zero")
        dsize *= zsize
    sp = get_sequence_parallel_size()
    if sp > 1:
        if dsize % sp != 0:
            logger.error("data parallel size %d should be divisible by sequence parallel size %d", dsize, sp)
        dsize //= sp
        drank //= sp
    return drank, dsize


# --------------------------------------------------------------------------------------------
# sequence parallel (Ulysses) helpers
# --------------------------------------------------------------------------------------------
def create_sequence_parallel_group(sp_size: int):
    if sp_size <= 1:
        return None
    ws = world_size()
    if ws % sp_size != 0:
        logger.error("World size %d is not divisible by sequence parallel size %d", ws, sp_size)
    _register(_SP_NAME, sp_size, [list(range(i, i + sp_size)) for i in range(0, ws, sp_size)])
    return parallel_group(_SP_NAME)


def destroy_sequence_parallel_group() -> None:
    pn = _pname(_SP_NAME)
    for g, _ in _S.groups_and_ranks.pop(pn, []):
        if g is not None:
            dist.destroy_process_group(g)
            if g in _S.owned_groups:
                _S.owned_groups.remove(g)
    _S.group.pop(pn, None)
    _S.group_rank.pop(pn, None)
    _S.group_size.pop(pn, None)


def get_sequence_parallel_group():
    return parallel_group(_SP_NAME)


def get_sequence_parallel_size() -> int:
    return parallel_group_size(_SP_NAME) or 1


def get_sequence_parallel_rank() -> int:
    return parallel_rank(_SP_NAME) or 0


class _SeqAllToAll(torch.autograd.Function):
    """Scatter dim ``scatter_idx`` over the group and gather dim ``gather_idx`` (one all-to-all);
    the backward is the inverse exchange."""

    @staticmethod
    def forward(ctx, x, scatter_idx, gather_idx, group, sp_size):
        sp_size = sp_size or dist.get_world_size(group)
        ctx.cfg = (scatter_idx, gather_idx, group, sp_size)
        if sp_size == 1:
            return x
        # [.., scatter, ..] -> [sp, .., scatter/sp, ..] contiguous chunks, one per destination
        send = torch.stack([c for c in torch.tensor_split(x, sp_size, scatter_idx)]).contiguous()
        grp = group if group is not None else dist.group.WORLD
        if send.is_cuda and os.environ.get("ATB_FUSED_COMM", "1") != "0":
            from ..parallel import symm

            if sp_size == dist.get_world_size(grp) and symm.all_to_all_available(send, grp):
                recv = symm.all_to_all_pull(send, grp)      # copy-engine pulls out of symmetric memory
                return torch.cat(list(recv.unbind(0)), dim=gather_idx).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return torch.cat(list(recv.unbind(0)), dim=gather_idx).contiguous()

    @staticmethod
    def backward(ctx, g):
        scatter_idx, gather_idx, group, sp_size = ctx.cfg
        return _SeqAllToAll.apply(g, gather_idx, scatter_idx, group, sp_size), None, None, None, None


def seq_all_to_all(input: torch.Tensor, scatter_idx: int, gather_idx: int, group=None, group_size=None):
    return _SeqAllToAll.apply(input, scatter_idx, gather_idx, group, group_size)


# --------------------------------------------------------------------------------------------
# init / reset
# --------------------------------------------------------------------------------------------
def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _env_defaults() -> None:
    env = os.environ
    env.setdefault("RANK", "0")
    env.setdefault("LOCAL_RANK", env["RANK"])
    env.setdefault("WORLD_SIZE", "1")
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in env:
        env["MASTER_PORT"] = str(find_free_port()) if env["WORLD_SIZE"] == "1" else "29500"
    if "NPROC_PER_NODE" not in env:
        env["NPROC_PER_NODE"] = env.get("LOCAL_WORLD_SIZE", "1" if env["WORLD_SIZE"] == "1" else env["WORLD_SIZE"])
    env.setdefault("NODE_SIZE", str(max(int(env["WORLD_SIZE"]) // int(env["NPROC_PER_NODE"]), 1)))
    env.setdefault("COWORKER_SIZE", "0")


_BACKENDS = ("nccl", "gloo", "cpu:gloo,cuda:nccl")


def init_distributed(backend: str = "nccl", coworker_num_per_node: int = 0, elastic_or_fault_tolerant: bool = False,
                     set_cuda_device_using_local_rank: bool = False, timeout=None, **kwargs) -> bool:
    """Initialise ``torch.distributed`` from the launcher environment (RANK, LOCAL_RANK, WORLD_SIZE,
    MASTER_ADDR, MASTER_PORT, NPROC_PER_NODE | LOCAL_WORLD_SIZE, NODE_SIZE); missing variables default
    to a single-process job. ``nccl`` without a GPU falls back to ``gloo``. The collective timeout
    can also be set with ``ATORCH_NCCL_EXEC_TIMEOUT`` (seconds). Returns True on success."""
    backend = backend.lower()
    if backend not in _BACKENDS:
        logger.error("Invalid backend %s. Only support %s", backend, _BACKENDS)
        return False
    if "nccl" in backend and not torch.cuda.is_available():
        logger.warning("no CUDA device: using gloo instead of %s", backend)
        backend = "gloo"
    _env_defaults()
    env = os.environ
    _S.rank, _S.local_rank, _S.world_size = int(env["RANK"]), int(env["LOCAL_RANK"]), int(env["WORLD_SIZE"])
    _S.nproc_per_node, _S.node_size = int(env["NPROC_PER_NODE"]), int(env["NODE_SIZE"])
    _S.coworker_size = int(env["COWORKER_SIZE"])
    if timeout is None:
        secs = env.get("ATORCH_NCCL_EXEC_TIMEOUT")
        timeout = datetime.timedelta(seconds=int(secs)) if secs else datetime.timedelta(minutes=30)
    if set_cuda_device_using_local_rank and torch.cuda.is_available():
        torch.cuda.set_device(_S.local_rank % torch.cuda.device_count())
    if not dist.is_initialized():
        pg_kwargs = {}
        if "nccl" in backend and torch.cuda.is_available():
            pg_kwargs["device_id"] = torch.device("cuda", _S.local_rank % torch.cuda.device_count())
        try:
            dist.init_process_group(backend, init_method="env://", rank=_S.rank, world_size=_S.world_size,
                                    timeout=timeout, **pg_kwargs)
        except Exception as e:  # pragma: no cover - depends on the environment
            logger.error("init_process_group failed: %s", e)
            return False
    _S.backend = backend
    _S.initialized = True
    return True


def reset_distributed() -> None:
    """Destroy every group created here and the default process group."""
    if not _S.initialized and not (dist.is_available() and dist.is_initialized()):
        return
    destroy_parallel_group()
    if dist.is_initialized():
        dist.destroy_process_group()
    _S.__init__()
