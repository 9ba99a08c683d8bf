"""ZeRO family: ``zero1`` (sharded optimizer state), ``zero2`` (+ sharded gradients), ``fsdp``
(ZeRO-3, parameters sharded too) and ``fsdp2`` (same engine, per-module mesh style config).

All four run on the native sharded engine (:mod:`atorch_b200.parallel.fsdp`): ``zero2`` keeps the
parameters gathered between forward and backward (``reshard_after_forward=False``), ``zero1`` is
``zero2`` with one whole-model unit. Unlike the reference (which raises "FSDP only support GPU",
atorch/auto/opt_lib/zero_optimization.py:316-317) the engine also runs on CPU with gloo.

Accepted ``fsdp`` config keys (reference: zero_optimization.py:302-502): ``atorch_wrap_cls``
(classes or class names), ``atorch_size_based_min_num_params`` (default 1e5 when no wrap class),
``atorch_ignored_cls``, ``sync_module_states``, ``forward_prefetch``, ``backward_prefetch``,
``limit_all_gathers``, ``use_orig_params``, ``cpu_offload``, ``param_init_fn``, ``mixed_precision``
(object with ``param_dtype``/``reduce_dtype``), ``sharding_strategy``, ``use_local_sgd`` with
``local_sgd_config`` / ``outer_optim_config`` / ``gta_config``.
"""
from __future__ import annotations

import logging

import torch

from ...distributed import distributed as D
from .optimization import Optimization

logger = logging.getLogger("atorch.logger")

_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32,
           "float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def _to_dtype(d):
    if d is None or isinstance(d, torch.dtype):
        return d
    return _DTYPES[str(d)]


def build_sharded_model(model_context, cfg: dict, reshard_after_forward: bool = True, single_unit: bool = False):
    from ...parallel.fsdp import FSDP, ShardingConfig

    cfg = dict(cfg or {})
    wrap_cls = cfg.pop("atorch_wrap_cls", None)
    min_params = cfg.pop("atorch_size_based_min_num_params", None)
    ignored_cls = cfg.pop("atorch_ignored_cls", None)
    if single_unit:
        wrap_cls, min_params = None, None
    elif wrap_cls is None and min_params is None:
        min_params = int(1e5)
    mp = cfg.pop("mixed_precision", None)
    param_dtype = _to_dtype(cfg.pop("param_dtype", None))
    reduce_dtype = _to_dtype(cfg.pop("reduce_dtype", None))
    if mp is not None:
        get = mp.get if isinstance(mp, dict) else (lambda k, d=None: getattr(mp, k, d))
        param_dtype = _to_dtype(get("param_dtype")) or param_dtype
        reduce_dtype = _to_dtype(get("reduce_dtype")) or reduce_dtype
    strategy = str(cfg.pop("sharding_strategy", "") or "")
    if "SHARD_GRAD_OP" in strategy:
        reshard_after_forward = False
    group = cfg.pop("process_group", None)
    replica = cfg.pop("replica_group", None)
    if group is None:
        group = D.parallel_group("zero") or D.parallel_group("data")
    device = cfg.pop("device_id", None)
    if isinstance(device, int):
        device = torch.device("cuda", device)
    if device is None and torch.cuda.is_available() and (D.backend() is None or "nccl" in (D.backend() or "")):
        device = torch.device("cuda", torch.cuda.current_device())
    sc = ShardingConfig(
        process_group=group, replica_group=replica, param_dtype=param_dtype, reduce_dtype=reduce_dtype,
        reshard_after_forward=cfg.pop("reshard_after_forward", reshard_after_forward),
        forward_prefetch=cfg.pop("forward_prefetch", True),
        backward_prefetch=bool(cfg.pop("backward_prefetch", True)),
        sync_module_states=cfg.pop("sync_module_states", False),
        param_init_fn=cfg.pop("param_init_fn", None), device=device,
        checkpoint_units=cfg.pop("checkpoint_units", False), fused_comm=cfg.pop("fused_comm", None),
        optimizer_in_backward=cfg.pop("optimizer_in_backward", False), comm_blocks=cfg.pop("comm_blocks", 32),
        prefetch_depth=int(cfg.pop("prefetch_depth", 2)))
    # torch FSDP's limit_all_gathers (a rate limiter of in-flight all-gathers) maps onto the bounded
    # prefetch depth of this engine: at most prefetch_depth + 1 units are ever gathered at once
    cfg.pop("limit_all_gathers", None)
    use_local_sgd = cfg.pop("use_local_sgd", False)
    lsgd = {k: cfg.pop(k, None) for k in ("local_sgd_config", "outer_optim_config", "gta_config")}
    for k in ("use_orig_params", "cpu_offload", "auto_wrap_policy", "wrap_trainable_outmost",
              "intra_load", "fsdp_wrap_params_outmost", "backward_prefetch_policy", "ignored_modules",
              "keep_low_precision_grads"):
        cfg.pop(k, None)
    if cfg:
        logger.warning("fsdp: ignoring unknown config keys %s", sorted(cfg))
    model = FSDP(model_context.model, wrap_cls=wrap_cls, min_num_params=min_params, ignored_cls=ignored_cls,
                 config=sc)
    if use_local_sgd:
        from ...local_sgd.sharded import attach_local_sgd

        attach_local_sgd(model, lsgd["local_sgd_config"], lsgd["outer_optim_config"], lsgd["gta_config"])
    return model


def _fsdp_wrapper(model_context, wrapper_name, wrapper_config=None):
    model_context.model = build_sharded_model(model_context, wrapper_config, True)
    return model_context


def _zero2_wrapper(model_context, wrapper_name, wrapper_config=None):
    model_context.model = build_sharded_model(model_context, wrapper_config, False)
    return model_context


def _zero1_wrapper(model_context, wrapper_name, wrapper_config=None):
    model_context.model = build_sharded_model(model_context, wrapper_config, False, single_unit=True)
    return model_context


class FSDPOptimization(Optimization):
    def __init__(self, name="fsdp"):
        super().__init__(name, "zero", False, False)

    def transform(self, model_context, config=None):
        model_context.add_wrapper("fsdp", _fsdp_wrapper, dict(config or {}), is_pre_wrapper=True)
        return model_context


class FSDP2Optimization(FSDPOptimization):
    def __init__(self):
        super().__init__("fsdp2")

    def transform(self, model_context, config=None):
        cfg = dict(config or {})
        mp = cfg.get("mixed_precision")
        if isinstance(mp, dict):
            cfg["mixed_precision"] = mp
        model_context.add_wrapper("fsdp", _fsdp_wrapper, cfg, is_pre_wrapper=True)
        return model_context


class Zero2Optimization(Optimization):
    def __init__(self):
        super().__init__("zero2", "zero", False, False)

    def transform(self, model_context, config=None):
        cfg = dict(config or {})
        cfg.pop("not_use_fsdp", None)
        cfg.pop("use_ds_zero", None)
        model_context.add_wrapper("fsdp", _zero2_wrapper, cfg, is_pre_wrapper=True)
        return model_context


class Zero1Optimization(Optimization):
    def __init__(self):
        super().__init__("zero1", "zero", False, False)

    def transform(self, model_context, config=None):
        cfg = dict(config or {})
        cfg.pop("use_ds_zero", None)
        model_context.add_wrapper("fsdp", _zero1_wrapper, cfg, is_pre_wrapper=True)
        return model_context
