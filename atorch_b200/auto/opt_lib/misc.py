"""Smaller optimisation methods: ``native_dynamo``, ``sequence_parallel``, and the entry points of
``tensor_parallel`` / ``pipeline_parallel`` / ``mixed_parallel`` / ``fp8`` / ``deepspeed_3d_parallel``,
whose machinery lives in :mod:`atorch_b200.parallel` and :mod:`atorch_b200.modules`.

(Reference: atorch/auto/opt_lib/dynamo_optimization.py:10, sequence_parallel_optimization.py:9-103,
tensor_parallel_optimization.py:23-168, pipeline_parallel_optimization.py:56,
mixed_parallel_optimization.py:32-307, amp_optimization.py:216-521, ds_3d_parallel_optimization.py:62.)
"""
from __future__ import annotations

import logging

import torch

from ...distributed import distributed as D
from .optimization import Optimization

logger = logging.getLogger("atorch.logger")


def _dynamo_wrapper(model_context, wrapper_name, wrapper_config=None):
    """``torch.compile`` of the user model. Not used on this framework's own hot paths (those are
    hand-written kernels); offered because users of arbitrary models may ask for it."""
    cfg = dict(wrapper_config or {})
    model_context.model = torch.compile(model_context.model, **cfg)
    return model_context


class NativeDynamoOptimization(Optimization):
    def __init__(self):
        super().__init__("native_dynamo", "dynamo", False)

    def transform(self, model_context, config=None):
        model_context.add_wrapper("native_dynamo", _dynamo_wrapper, config, is_pre_wrapper=True)
        return model_context


def _sp_wrapper(model_context, wrapper_name, wrapper_config=None):
    cfg = dict(wrapper_config or {})
    sp_size = int(cfg.get("sp_size", 1))
    if sp_size <= 1:
        return model_context
    if D.get_sequence_parallel_group() is None:
        D.create_sequence_parallel_group(sp_size)
    group, rank = D.get_sequence_parallel_group(), D.get_sequence_parallel_rank()
    fn_name = cfg.get("set_sp_func_name", "set_sp")
    classes = cfg.get("module")
    if classes is not None and not isinstance(classes, (list, tuple)):
        classes = (classes,)
    for m in model_context.model.modules():
        if (classes is None and hasattr(m, fn_name)) or (classes is not None and isinstance(m, tuple(classes))):
            getattr(m, fn_name)(sp_size, rank, group)
    fn = cfg.get("batch_sp_processing_fn")
    if fn is not None:
        pi = model_context.prepare_input

        def prepare_input(batch, device):
            if pi is not None:
                batch = pi(batch, device)
            return fn(batch, sp_size, rank)
        model_context.prepare_input = prepare_input
    return model_context


class SequenceParallelOptimization(Optimization):
    def __init__(self):
        super().__init__("sequence_parallel", "sequence_parallel", False, True)

    def transform(self, model_context, config=None):
        model_context.add_wrapper("sequence_parallel", _sp_wrapper, config, is_pre_wrapper=True)
        return model_context


def _tp_wrapper(model_context, wrapper_name, wrapper_config=None):
    from ...parallel.tensor_parallel import apply_tensor_parallel

    model_context.model = apply_tensor_parallel(model_context.model, wrapper_config or {})
    model_context.update_tp_status(True)
    return model_context


class TensorParallelOptimization(Optimization):
    def __init__(self):
        super().__init__("tensor_parallel", "parallel", True, True)

    def tune(self, model_context, config=None, strategy=None, apply_transform=True, time_limit=None):
        from ...parallel.tensor_parallel import plan_tensor_parallel

        best = plan_tensor_parallel(model_context.model, config or {})
        if apply_transform:
            model_context = self.transform(model_context, best)
        return True, best, model_context

    def transform(self, model_context, config=None):
        model_context.add_wrapper("tp", _tp_wrapper, config, is_pre_wrapper=True)
        return model_context


def _fp8_wrapper(model_context, wrapper_name, wrapper_config=None):
    from ...modules.fp8 import convert_linears_to_fp8

    convert_linears_to_fp8(model_context.model, wrapper_config or {})
    return model_context


class Fp8Optimization(Optimization):
    def __init__(self):
        super().__init__("fp8", "amp", False)

    def device_supported(self, config=None, device_capability=None) -> bool:
        return device_capability is not None and tuple(device_capability) >= (8, 9)

    def transform(self, model_context, config=None):
        model_context.add_wrapper("fp8", _fp8_wrapper, config, is_pre_wrapper=True)
        return model_context


def _pipe_wrapper(model_context, wrapper_name, wrapper_config=None):
    from ...pipeline_parallel.auto_pipe import pipeline_model_context

    return pipeline_model_context(model_context, wrapper_config or {})


class PipelineParallelOptimization(Optimization):
    def __init__(self):
        super().__init__("pipeline_parallel", "parallel", True, True)

    def transform(self, model_context, config=None):
        model_context.add_wrapper("pipe", _pipe_wrapper, config, is_pre_wrapper=False)
        return model_context


class MixedParallelOptimization(Optimization):
    """Automatic tensor x pipeline x data split: sizes from ``parallel_mode`` or from the dim planner."""

    def __init__(self):
        super().__init__("mixed_parallel", "parallel", True, True)

    def tune(self, model_context, config=None, strategy=None, apply_transform=True, time_limit=None):
        from ...auto.planner import plan_mixed_parallel

        best = plan_mixed_parallel(model_context, config or {})
        if apply_transform:
            model_context = self.transform(model_context, best)
        return True, best, model_context

    def transform(self, model_context, config=None):
        cfg = dict(config or {})
        if cfg.get("tensor_parallel") is not None:
            model_context.add_wrapper("tp", _tp_wrapper, cfg["tensor_parallel"], is_pre_wrapper=True)
        if cfg.get("pipeline_parallel") is not None:
            model_context.add_wrapper("pipe", _pipe_wrapper, cfg["pipeline_parallel"], is_pre_wrapper=False)
        return model_context


class DeepSpeed3DParallelOptimization(Optimization):
    """3-D (tensor x pipeline x data) layout described by a ``TPInfo`` and a stage count: runs on
    the native tensor/pipeline runtimes (no DeepSpeed dependency)."""

    def __init__(self):
        super().__init__("deepspeed_3d_parallel", "parallel", False, True)

    def transform(self, model_context, config=None):
        from ...parallel.tensor_parallel import tp_config_from_3d

        tp_cfg, pipe_cfg = tp_config_from_3d(config)
        if tp_cfg is not None:
            model_context.add_wrapper("tp", _tp_wrapper, tp_cfg, is_pre_wrapper=True)
        if pipe_cfg is not None:
            model_context.add_wrapper("pipe", _pipe_wrapper, pipe_cfg, is_pre_wrapper=False)
        return model_context
