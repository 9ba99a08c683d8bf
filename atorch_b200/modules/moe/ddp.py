"""Data parallelism for models that mix dense and expert parameters.

Dense parameters are replicated on every rank of the data-parallel group and their gradients are averaged
over it. Expert parameters exist once per expert-parallel group; only the ranks that hold the *same*
experts (the "experts DDP" group, set with ``set_experts_ddp_process_group``; none when every rank has
its own experts) average them. ``MoEMixtureDistributedDataParallel`` runs one bucketed reducer of
:mod:`atorch_b200.parallel.ddp` per kind of parameter, both overlapped with the backward pass.

A parameter counts as an expert parameter when it belongs to an ``Experts`` / ``Grouped_GEMM_MoE`` module
or carries ``is_expert = True`` (or the older ``allreduce = False``) as an attribute.
(Reference: atorch/modules/moe/ddp.py:31-360, which rebuilds torch DDP's reducer for the expert group.)
"""
from __future__ import annotations

import contextlib
from typing import List, Optional, Set, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ...parallel.ddp import DistributedDataParallel

_EXPERTS_DDP_PG = {"group": None}


def set_experts_ddp_process_group(group) -> None:
    _EXPERTS_DDP_PG["group"] = group


def get_experts_ddp_process_group():
    return _EXPERTS_DDP_PG["group"]


def split_moe_and_dense_params(module: nn.Module) -> Tuple[List[str], List[str]]:
    """Names of the expert parameters and of the dense parameters of ``module``."""
    from .grouped_gemm_moe import Grouped_GEMM_MoE
    from .moe_layer import Experts

    moe: Set[str] = set()
    for mname, m in module.named_modules():
        if isinstance(m, (Experts, Grouped_GEMM_MoE)):
            for pname, _ in m.named_parameters():
                moe.add(f"{mname}.{pname}" if mname else pname)
    dense = []
    for n, p in module.named_parameters():
        if getattr(p, "is_expert", False) or getattr(p, "allreduce", True) is False:
            moe.add(n)
        if n not in moe:
            dense.append(n)
    return sorted(moe), dense


class _Empty:
    def _attach_views(self):
        pass


class MoEMixtureDistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, device_ids=None, output_device=None, dim=0, broadcast_buffers: bool = True,
                 process_group=None, bucket_cap_mb: float = 25, find_unused_parameters: bool = False,
                 check_reduction: bool = False, gradient_as_bucket_view: bool = False, static_graph: bool = False):
        super().__init__()
        self.module = module
        moe_names, dense_names = split_moe_and_dense_params(module)
        self.moe_params_names, self.dense_params_names = set(moe_names), set(dense_names)
        self.process_group = process_group
        self.experts_process_group = get_experts_ddp_process_group()
        self.dense = DistributedDataParallel(module, process_group, bucket_cap_mb, find_unused_parameters,
                                             broadcast_buffers, param_filter=lambda n, p: n in self.dense_params_names)
        self.experts = None
        if self.moe_params_names and self.experts_process_group is not None and \
                dist.get_world_size(self.experts_process_group) > 1:
            self.experts = DistributedDataParallel(module, self.experts_process_group, bucket_cap_mb,
                                                   find_unused_parameters, False,
                                                   param_filter=lambda n, p: n in self.moe_params_names)

    def forward(self, *args, **kwargs):
        if torch.is_grad_enabled():
            self.dense._attach_views()
            if self.experts is not None:
                self.experts._attach_views()
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        with contextlib.ExitStack() as st:
            st.enter_context(self.dense.no_sync())
            if self.experts is not None:
                st.enter_context(self.experts.no_sync())
            yield

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, *a, **k):
        return self.module.load_state_dict(*a, **k)
