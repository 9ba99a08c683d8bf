"""``PipeModuleConfig`` / ``PipeModule`` / ``make_pipe_module``: build this rank's pipeline stages.

``model_provider(model_config, layer_num, pre_process, post_process, start_layer_idx)`` returns the
module chunk of one stage; each chunk may get its own ``auto_accelerate`` strategy (plus ``auto_ddp``
over the ``data`` group), then is wrapped into a ``PipeStage``.
(Reference: atorch/pipeline_parallel/pipe_module.py:19-265.)
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch
import torch.nn as nn

from ..communication.pipe_communicator import PipeCommunicator
from ..distributed import distributed as D
from .pipe_partition import partition_model_from_model_provider
from .pipe_stage import PipeStage


class PipeModuleConfig:
    def __init__(self, partition_method="default", manual_stage_partition=None, model_config=None,
                 total_layer_num=None, tie_weight_info=None, input_output_mapping=None, virtual_pp_size=None,
                 auto_ddp=True, sche_name="Schedule1F1B", n_microbatches=1):
        self.partition_method, self.manual_stage_partition = partition_method, manual_stage_partition
        self.model_config, self.total_layer_num = model_config, total_layer_num
        self.tie_weight_info, self.input_output_mapping = tie_weight_info, input_output_mapping
        self.virtual_pp_size, self.auto_ddp = virtual_pp_size, auto_ddp
        self.sche_name, self.n_microbatches = sche_name, n_microbatches


class PipeModule(nn.Module):
    def __init__(self, modules: List[nn.Module], stage_ids: List[int], num_stages: int,
                 input_output_mapping: Optional[Dict], loss_func: Optional[Callable] = None, tie_weight_info=None,
                 strategy: Optional[Any] = None, auto_ddp: bool = True, device=None):
        super().__init__()
        assert len(modules) == len(stage_ids)
        self.stage_modules = nn.ModuleList(modules)
        self.stage_ids, self.num_stages = list(stage_ids), num_stages
        self.ori_loss_func = loss_func
        self.loss_func = loss_func if num_stages - 1 in stage_ids else None
        self.input_output_mapping = input_output_mapping
        self.virtual_pp_size = len(stage_ids)
        self.pp_size = D.parallel_group_size("pipe") or 1
        self.pp_rank = D.parallel_rank("pipe") or 0
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if (
                torch.cuda.is_available() and "nccl" in (D.backend() or "")) else torch.device("cpu")
        self.device = device
        self._apply_strategy(strategy, auto_ddp)
        self.stages = self._create_stages()

    def _apply_strategy(self, strategy, auto_ddp):
        from ..auto.accelerate import auto_accelerate

        mods = []
        for i, m in enumerate(self.stage_modules):
            st = strategy[i] if isinstance(strategy, tuple) else strategy
            st = list(st) if st is not None else []
            if auto_ddp and D.parallel_group("data") is not None and (D.parallel_group_size("data") or 1) > 1 \
                    and not any((s if isinstance(s, str) else s[0]) in ("fsdp", "zero1", "zero2", "fsdp2") for s in st):
                st = st + ["auto_ddp"]
            if st:
                ok, res, _ = auto_accelerate(m, load_strategy=st, ignore_dryrun_on_load_strategy=True)
                assert ok, "applying the stage strategy failed"
                m = res.model
            else:
                m = m.to(self.device)
            mods.append(m)
        self.stage_modules = nn.ModuleList(mods)

    def _create_stages(self) -> List[PipeStage]:
        group = D.parallel_group("pipe")
        _, ranks = D.parallel_group_and_ranks("pipe")
        ranks = ranks or [D.rank() or 0]
        comm = PipeCommunicator(group, self.device) if self.pp_size > 1 else None
        pp_size = self.pp_size

        def stage_to_rank(sid):
            return ranks[sid % pp_size] if self._style() == "loop" else ranks[min(sid, self.num_stages - 1 - sid)]
        return [PipeStage(m, sid, self.num_stages, self.device, self.input_output_mapping, comm, stage_to_rank,
                          D.rank() if D.rank() is not None else 0)
                for m, sid in zip(self.stage_modules, self.stage_ids)]

    def _style(self):
        ids = self.stage_ids
        if len(ids) == 2 and ids[1] == self.num_stages - 1 - ids[0] and ids[1] != ids[0] + self.pp_size:
            return "v"
        return "loop"

    def parameters(self, recurse: bool = True):
        for m in self.stage_modules:
            yield from m.parameters()

    def forward(self, *a, **k):
        raise RuntimeError("a PipeModule is driven by a pipeline schedule (make_pipe_schedule_from_pipe_module)")


def make_pipe_module(meta_model=None, model_provider=None, loss_func=None, strategy=None, distributed_context=None,
                     config: Optional[PipeModuleConfig] = None) -> PipeModule:
    assert config is not None, "config is required"
    ctx = distributed_context or D
    if model_provider is not None:
        modules, stage_ids, tie = partition_model_from_model_provider(model_provider, ctx, config)
    else:
        assert meta_model is not None, "give a model_provider or a (meta) model"
        from .pipe_partition import partition_model_from_meta_model

        modules, stage_ids, tie = partition_model_from_meta_model(meta_model, ctx, config)
    total = (ctx.parallel_group_size("pipe") or 1) * (config.virtual_pp_size or 1)
    return PipeModule(modules, stage_ids, total, config.input_output_mapping, loss_func, tie, strategy,
                      config.auto_ddp)
