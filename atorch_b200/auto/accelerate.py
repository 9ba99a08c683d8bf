"""``auto_accelerate``: apply an acceleration strategy to a plain PyTorch training job.

    status, result, best_strategy = auto_accelerate(model, optim_func, dataset, loss_func,
                                                    prepare_input, model_input_format, optim_args,
                                                    load_strategy=[...])

``result`` is ``AutoAccelerateResult(model, optim, dataloader, loss_func, prepare_input,
lr_scheduler, args)``; the caller then runs an ordinary loop on those objects
(``loss.backward()`` unless ``result.args["use_optim_backward"]``).

* With ``load_strategy`` (a list of names or ``(name, config)`` pairs, a ``Strategy``, pickled bytes
  or a file name) the strategy is validated, adjusted to the running world size, its tunable
  entries tuned, optionally dry-run, and applied.
* Without it the acceleration engine searches: candidate strategies are generated, dry-run
  (throughput, peak memory) and the best one is applied (:mod:`atorch_b200.auto.engine`).

Extra keyword arguments: ``verbose, time_limit, find_unused_parameters, sample_batch, batch_size,
expand_sample_batch, sampler_seed, ignore_dryrun_on_load_strategy (default True),
meta_init_offload_name``.

(Reference: atorch/auto/accelerate.py:34-86 ``model_transform``, :267-323 ``get_strategy`` /
``save_strategy``, :326-380 ``adjust_strategy``, :427-660 ``auto_accelerate``.)
"""
from __future__ import annotations

import collections
import logging
import os
import pickle
from typing import Optional

import torch

from ..distributed import distributed as D
from .auto_accelerate_context import AutoAccelerateContext
from .device_context import get_device_context
from .model_context import ModelContext
from .opt_lib.optimization_library import SEMIAUTO_STRATEGIES, OptimizationLibrary
from .opt_lib.parallel_mode import ParallelModeOptimization
from .strategy import Strategy

logger = logging.getLogger("atorch.logger")

AutoAccelerateResult = collections.namedtuple(
    "AutoAccelerateResult", "model, optim, dataloader, loss_func, prepare_input, lr_scheduler, args")

EXTRA_ARGS = ("verbose", "time_limit", "find_unused_parameters", "sample_batch", "batch_size",
              "expand_sample_batch", "sampler_seed", "ignore_dryrun_on_load_strategy", "meta_init_offload_name",
              "disable_fused_optimizer", "optim_param_func_args")


def assemble_result(mc: ModelContext) -> AutoAccelerateResult:
    return AutoAccelerateResult(mc.model, mc.optim, mc.dataloader, mc.loss_func, mc.prepare_input, mc.lr_scheduler,
                                mc.args)


def get_strategy(load_strategy):
    """(status, Strategy) from a file name, pickled bytes, a ``Strategy`` or a list of entries."""
    try:
        if isinstance(load_strategy, Strategy):
            return True, load_strategy
        if isinstance(load_strategy, str):
            with open(load_strategy, "rb") as f:
                load_strategy = f.read()
        if isinstance(load_strategy, bytes):
            return True, Strategy.loads(load_strategy)
        if isinstance(load_strategy, (list, tuple)):
            s = Strategy()
            for item in load_strategy:
                if isinstance(item, str):
                    s.add_opt((item, None, None))
                elif isinstance(item, (tuple, list)) and len(item) == 2:
                    s.add_opt((item[0], item[1], item[0] in SEMIAUTO_STRATEGIES and item[1] is None))
                elif isinstance(item, (tuple, list)) and len(item) == 3:
                    s.add_opt(tuple(item))
                else:
                    raise ValueError("load_strategy list items must be a name or (name, config)")
            return True, s
        raise ValueError("load_strategy must be a file name, bytes, a Strategy or a list")
    except Exception as e:
        logger.error("cannot load strategy: %s", e)
        return False, None


def save_strategy(strategy: Strategy, filename: str) -> None:
    with open(filename, "wb") as f:
        f.write(pickle.dumps(strategy))


def adjust_strategy(strategy: Strategy, device_context, finetune_strategy: bool, opt_lib: OptimizationLibrary):
    """Fit the strategy to the running job: rescale the ``data`` dim to the world size, drop
    distributed-only methods in a single-process run and methods the device cannot run."""
    found, pmode = strategy.get_parallel_mode()
    world = D.world_size() or 1
    if pmode is not None:
        total, dsize, has_data = 1, 1, False
        for n, s in pmode[0]:
            total *= s
            if n == "data":
                dsize, has_data = s, True
        multi = pmode[2] if len(pmode) > 2 else False
        if total != world and not multi:
            if pmode[1] is not None or not has_data or (world * dsize) % total != 0:
                logger.error("strategy needs %d processes (data=%d), job has %d", total, dsize, world)
                return False, None
            strategy.adjust_data_parallel(world * dsize // total)
    elif found:
        strategy.adjust_data_parallel(world)
    if not D.is_distributed():
        removed = strategy.remove_distributed_method(opt_lib)
        if removed:
            logger.info("ignored in a single-process run: %s", removed)
    cap = torch.cuda.get_device_capability() if torch.cuda.is_available() else None
    removed = strategy.remove_device_unsupported_method(opt_lib, cap)
    if removed:
        logger.info("ignored, not supported by this device: %s", removed)
    if finetune_strategy:
        strategy.reset_config()
    strategy.set_tunable_value(opt_lib)
    return True, strategy


def model_transform(model_context: ModelContext, strategy: Strategy, opt_lib: OptimizationLibrary,
                    create_optim: bool = True, create_dataloader: bool = True) -> ModelContext:
    """Register every method's wrappers, then build: pre-wrappers -> dataloader -> optimizer -> post-wrappers."""
    for name, config, _ in strategy:
        model_context = opt_lib[name].transform(model_context, config)
    model_context.adjust_wrappers()
    model_context.apply_wrappers(is_pre_wrapper=True)
    if create_dataloader:
        model_context.update_dataloader()
    if create_optim:
        model_context.update_optim()
    model_context.apply_wrappers(is_pre_wrapper=False)
    from ..parallel.fsdp import FSDP

    model = model_context.model
    if not isinstance(model, FSDP) and torch.cuda.is_available() and isinstance(model, torch.nn.Module):
        p = next(model.parameters(), None)
        if p is not None and p.device.type == "cpu" and (D.backend() is None or "nccl" in (D.backend() or "")):
            model_context.model = model.to(torch.device("cuda", torch.cuda.current_device()))
    return model_context


def tune_strategy(model_context: ModelContext, strategy: Strategy, opt_lib: OptimizationLibrary, time_limit=None):
    """Run ``tune`` of every tunable entry (they fill in their own config)."""
    for entry in strategy.opt_list:
        name, config, tunable = entry
        if tunable:
            ok, best, _ = opt_lib[name].tune(model_context, config, strategy, apply_transform=False,
                                             time_limit=time_limit)
            if not ok:
                return False
            entry[1], entry[2] = best, False
    return True


def auto_accelerate(model, optim_func=None, dataset=None, loss_func=None, prepare_input=None,
                    model_input_format=None, optim_args=None, optim_param_func=None, dataloader_args=None,
                    distributed_sampler_cls=None, excluded=None, included=None, load_strategy=None,
                    lr_scheduler_cls=None, lr_scheduler_args=None, finetune_strategy=False,
                    save_strategy_to_file=None, **kargs):
    extra = {k: kargs.pop(k) for k in list(kargs) if k in EXTRA_ARGS}
    if kargs:
        logger.warning("auto_accelerate: unknown arguments ignored: %s", sorted(kargs))
    AutoAccelerateContext.counter += 1
    mc = ModelContext(model=model, optim_func=optim_func, dataset=dataset, loss_func=loss_func,
                      prepare_input=prepare_input, model_input_format=model_input_format, optim_args=optim_args,
                      optim_param_func=optim_param_func, dataloader_args=dataloader_args,
                      distributed_sampler_cls=distributed_sampler_cls, lr_scheduler_cls=lr_scheduler_cls,
                      lr_scheduler_args=lr_scheduler_args, extra_args=extra)
    opt_lib = OptimizationLibrary()
    if load_strategy is None:
        from .engine import search as engine_search

        # the engine as a service on rank 0 (every rank is a client), or in-process when gRPC is not
        # importable or ATORCH_ENGINE_IN_PROCESS=1
        use_service = os.environ.get("ATORCH_ENGINE_IN_PROCESS", "0") != "1"
        if use_service:
            try:
                import grpc  # noqa: F401
            except ImportError:
                use_service = False
        fn = engine_search.search_strategy_with_service if use_service else engine_search.search_strategy
        ok, strategy = fn(mc, opt_lib, excluded=excluded, included=included, time_limit=extra.get("time_limit"),
                          verbose=extra.get("verbose", False))
        if not ok:
            return False, None, None
    else:
        ok, strategy = get_strategy(load_strategy)
        if not ok:
            return False, None, None
        ok, bad = opt_lib.validate_strategy(strategy)
        if not ok:
            logger.error("unknown optimisation methods: %s", bad)
            return False, None, None
        ok, strategy = adjust_strategy(strategy, get_device_context(), finetune_strategy, opt_lib)
        if not ok:
            return False, None, None
    _, pmode = strategy.get_parallel_mode()
    if pmode is not None and D.is_distributed():
        ParallelModeOptimization.setup_groups(pmode)
    if strategy.is_tunable():
        if not tune_strategy(mc, strategy, opt_lib, extra.get("time_limit")):
            return False, None, None
    if load_strategy is not None and not extra.get("ignore_dryrun_on_load_strategy", True):
        from .dry_runner import dry_run_strategy

        res = dry_run_strategy(mc, strategy, opt_lib)
        if res is None or res.get("throughput", 0) <= 0:
            logger.error("dry run of the loaded strategy failed")
            return False, None, None
    mc = model_transform(mc, strategy, opt_lib)
    if save_strategy_to_file:
        save_strategy(strategy, save_strategy_to_file)
    return True, assemble_result(mc), strategy
