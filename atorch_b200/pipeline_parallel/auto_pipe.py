"""Turning a whole-model ``ModelContext`` into a pipeline job (``pipeline_parallel`` optimisation).

The model must be a sequence of stages to cut: an ``nn.Sequential`` or a module exposing
``pipeline_layers()`` (a list of callables applied in order). Layers are split by
``stage_layers`` / evenly, this rank keeps its chunk, and ``model_context.model`` becomes a
``PipelinedModel`` whose ``forward(batch)`` runs the configured schedule and returns the loss.
(Reference: atorch/auto/opt_lib/pipeline_parallel_optimization.py:56-149, which compiles with PiPPy.)
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..distributed import distributed as D
from .pipe_module import PipeModule, PipeModuleConfig
from .pipe_partition import get_rank_stage_info
from .pipe_schedule import make_pipe_schedule_from_pipe_module


class PipelinedModel(nn.Module):
    def __init__(self, pipe_module: PipeModule, config: PipeModuleConfig):
        super().__init__()
        self.pipe_module = pipe_module
        self.schedule = make_pipe_schedule_from_pipe_module(pipe_module, config)
        self.first = 0 in pipe_module.stage_ids
        self.last = (pipe_module.num_stages - 1) in pipe_module.stage_ids

    def parameters(self, recurse: bool = True):
        return self.pipe_module.parameters()

    def forward(self, inputs=None, target=None):
        args = (inputs,) if (self.first and inputs is not None) else ()
        return self.schedule.step(*args, target=target if self.last else None)


def pipeline_model_context(model_context, config: Optional[dict] = None):
    config = dict(config or {})
    model = model_context.model
    layers = list(model.pipeline_layers()) if hasattr(model, "pipeline_layers") else list(model.children())
    pp = D.parallel_group_size("pipe") or 1
    rank = D.parallel_rank("pipe") or 0
    vpp = config.get("virtual_pp_size") or 1
    info = get_rank_stage_info(len(layers), rank, pp, vpp, manual_stage_partition=config.get("stage_layers"))
    chunks = [nn.Sequential(*layers[start: start + n]) for _, n, start in info]
    cfg = PipeModuleConfig(total_layer_num=len(layers), virtual_pp_size=vpp,
                           sche_name=config.get("sche_name", config.get("pipe_schedule", "Schedule1F1B")),
                           n_microbatches=config.get("n_microbatches", config.get("chunks", max(pp, 1))),
                           input_output_mapping=config.get("input_output_mapping"))
    loss = None
    if model_context.loss_func is not None:
        lf = model_context.loss_func
        loss = lambda out, tgt: lf(tgt, out)      # noqa: E731  (loss_func(batch, outputs) convention)
    pm = PipeModule(chunks, [s for s, _, _ in info], pp * vpp, cfg.input_output_mapping, loss, None,
                    config.get("stage_strategy"), config.get("auto_ddp", True))
    model_context.model = PipelinedModel(pm, cfg)
    return model_context
