"""``parallel_mode`` / ``auto_ddp``: create the named process groups and add data parallelism.

(Reference: atorch/auto/opt_lib/parallel_mode_optimization.py:10-62.)
"""
from __future__ import annotations

import torch

from ...distributed import distributed as D
from ...parallel.ddp import DistributedDataParallel
from .optimization import Optimization


def _ddp_wrapper(model_context, wrapper_name, wrapper_config=None):
    from ...parallel.fsdp import FSDP

    if isinstance(model_context.model, FSDP):
        return model_context
    group = D.parallel_group("data")
    if group is None or (D.parallel_group_size("data") or 1) <= 1:
        return model_context
    model = model_context.model
    if torch.cuda.is_available() and (D.backend() or "").find("nccl") >= 0:
        model = model.to(torch.device("cuda", D.local_rank()))
    model_context.model = DistributedDataParallel(
        model, process_group=group, find_unused_parameters=model_context.find_unused_parameters())
    return model_context


class ParallelModeOptimization(Optimization):
    def __init__(self):
        super().__init__("parallel_mode", "parallel_mode", False, True)

    def transform(self, model_context, config=None):
        model_context.parallel_mode_config = config
        if config is not None and any(n == "data" for n, _ in config[0]):
            model_context.add_wrapper("ddp", _ddp_wrapper, None, is_pre_wrapper=False)
        return model_context

    @staticmethod
    def setup_groups(config) -> None:
        """Create the groups of ``config`` unless an identical config is already active."""
        if config is None:
            return
        cur = D.parallel_config()
        if cur is not None and [tuple(x) for x in cur[0]] == [tuple(x) for x in config[0]]:
            return
        if cur is not None:
            D.destroy_parallel_group()
        D.create_parallel_group(config)


class AutoDDPOptimization(Optimization):
    """DDP over an already existing ``data`` group (used by pipeline stages)."""

    def __init__(self):
        super().__init__("auto_ddp", "parallel_mode", False, True)

    def transform(self, model_context, config=None):
        model_context.add_wrapper("ddp", _ddp_wrapper, None, is_pre_wrapper=False)
        return model_context
