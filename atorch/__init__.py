"""Import-path compatibility namespace: ``import atorch`` / ``from atorch.auto import auto_accelerate`` etc.
resolve to the modules of ``atorch_b200``. A meta-path finder maps ``atorch.<path>`` to
``atorch_b200.<path>`` with a small rename table for modules that live under a different name here.
An ``atorch_addon`` module, if importable, is loaded at import time unless ``ATORCH_DISABLE_ADDON`` is set
(as in the original package's ``__init__``)."""
import importlib
import importlib.abc
import importlib.util
import os
import sys

import atorch_b200
from atorch_b200 import coworker_size, init_distributed, local_rank, rank, reset_distributed, world_size  # noqa: F401

__version__ = atorch_b200.__version__

_RENAMES = {
    "atorch.auto.opt_lib.module_replace_optimization": "atorch_b200.auto.opt_lib.module_replace",
    "atorch.auto.opt_lib.zero_optimization": "atorch_b200.auto.opt_lib.zero",
    "atorch.auto.opt_lib.amp_optimization": "atorch_b200.auto.opt_lib.amp",
    "atorch.auto.opt_lib.checkpoint_optimization": "atorch_b200.auto.opt_lib.checkpoint",
    "atorch.auto.opt_lib.parallel_mode_optimization": "atorch_b200.auto.opt_lib.parallel_mode",
    "atorch.local_sgd.configs": "atorch_b200.local_sgd",
    "atorch.local_sgd.configs.configs": "atorch_b200.local_sgd.configs",
    "atorch.local_sgd.DDP": "atorch_b200.local_sgd",
    "atorch.local_sgd.DDP.outer_optim_model_averager": "atorch_b200.local_sgd.averager",
    "atorch.local_sgd.DDP.stateful_post_localSGD_optimizer": "atorch_b200.local_sgd.averager",
    "atorch.local_sgd.utils": "atorch_b200.local_sgd",
    "atorch.local_sgd.utils.anomaly_detection": "atorch_b200.local_sgd.anomaly",
    "atorch.local_sgd.utils.reduce_methods": "atorch_b200.local_sgd",
    "atorch.local_sgd.utils.reduce_methods.base": "atorch_b200.local_sgd.reducers",
    "atorch.local_sgd.utils.reduce_methods.linear": "atorch_b200.local_sgd.reducers",
    "atorch.local_sgd.utils.reduce_methods.generalized_task_arithmetic": "atorch_b200.local_sgd.reducers",
    "atorch.local_sgd.utils.reduce_methods.sparsify": "atorch_b200.local_sgd.reducers",
    "atorch.auto.engine.acceleration_engine": "atorch_b200.auto.engine.service",
    "atorch.auto.engine.servicer": "atorch_b200.auto.engine.service",
    "atorch.auto.task": "atorch_b200.auto.engine.task",
    "atorch.auto.engine.sg_algo.sg_algorithm": "atorch_b200.auto.engine.sg_algo",
    "atorch.auto.engine.sg_algo.sg_algo_lib": "atorch_b200.auto.engine.sg_algo",
    "atorch.auto.engine.sg_algo.combination_sg": "atorch_b200.auto.engine.sg_algo",
    "atorch.auto.engine.sg_algo.bayes_opt_sg": "atorch_b200.auto.engine.sg_algo",
    "atorch.auto.opt_lib.dynamo_optimization": "atorch_b200.auto.opt_lib.misc",
    "atorch.auto.opt_lib.mixed_parallel_optimization": "atorch_b200.auto.opt_lib.misc",
    "atorch.auto.opt_lib.sequence_parallel_optimization": "atorch_b200.auto.opt_lib.misc",
    "atorch.auto.opt_lib.tensor_parallel_optimization": "atorch_b200.auto.opt_lib.misc",
    "atorch.auto.opt_lib.half_optimization": "atorch_b200.auto.opt_lib.optimization_library",
    "atorch.auto.opt_lib.shard_planners": "atorch_b200.auto",
    "atorch.auto.opt_lib.shard_planners.dim_planner": "atorch_b200.auto.planner",
    "atorch.auto.opt_lib.shard_planners.mip_tp_planner": "atorch_b200.auto.mip_tp_planner",
    "atorch.distributed.mesh": "atorch_b200.distributed",
    "atorch.pipeline_parallel.scheduler": "atorch_b200.pipeline_parallel.pipe_engine",
    "atorch.modules.distributed_modules.randomizer": "atorch_b200.parallel.randomizer",
    "atorch.modules.distributed_modules.materialize_modules": "atorch_b200.utils.meta_model_utils",
    "atorch.optimizers.low_bit.optim.q_adamw": "atorch_b200.optimizers.low_bit.optim",
    "atorch.optimizers.low_bit.optim.q_agd": "atorch_b200.optimizers.low_bit.optim",
    "atorch.optimizers.low_bit.optim.q_came": "atorch_b200.optimizers.low_bit.optim",
    "atorch.optimizers.low_bit.optim.q_adafactor": "atorch_b200.optimizers.low_bit.optim",
    "atorch.rl.ppo_utils": "atorch_b200.rl",
    "atorch.rl.ppo_utils.ppo_util": "atorch_b200.rl.ppo_util",
    "atorch.rl.model_utils": "atorch_b200.rl",
    "atorch.rl.model_utils.model_util": "atorch_b200.rl.model_util",
    "atorch.rl.replay_buffer": "atorch_b200.rl",
    "atorch.rl.replay_buffer.replay_buffer": "atorch_b200.rl.trainer",
    "atorch.rl.trainer": "atorch_b200.rl",
    "atorch.rl.trainer.ppo_trainer": "atorch_b200.rl.trainer",
    "atorch.trainer.base.atorch_train_engine": "atorch_b200.trainer.engine",
    "atorch.local_sgd.FSDP": "atorch_b200.local_sgd.sharded",
    "atorch.modules.moe.topk_gating": "atorch_b200.modules.moe.prototype_gating",
    "atorch.modules.moe.switch_gating": "atorch_b200.modules.moe.prototype_gating",
    "atorch.modules.normalization.layernorm": "atorch_b200.modules.normalization",
    "atorch.optimizers.low_bit.optim": "atorch_b200.optimizers.low_bit",
    "atorch.trainer.atorch_trainer_v2": "atorch_b200.trainer.atorch_trainer_v2",
    "atorch.trainer.fsdp.fsdp_shard_async_saver": "atorch_b200.trainer.fsdp.fsdp_ckpt_saver",
    "atorch.trainer.fsdp.fsdp_shard_dcp_loader": "atorch_b200.trainer.fsdp.fsdp_ckpt_saver",
    "atorch.trainer.base": "atorch_b200.trainer",
    "atorch.trainer.base.dist_checkpointing": "atorch_b200.trainer",
    "atorch.trainer.base.dist_checkpointing.strategies": "atorch_b200.trainer",
    "atorch.trainer.base.dist_checkpointing.strategies.async_utils": "atorch_b200.trainer.async_calls",
    "atorch.trainer.megatron": "atorch_b200.trainer",
    "atorch.trainer.megatron.megatron_async_save": "atorch_b200.trainer.async_calls",
    "atorch.utils.numberic_checker": "atorch_b200.utils.numeric_checker",
    "atorch.utils.dynamic_profiler": "atorch_b200.utils.dynamic_profiler",
    "atorch.utils.inspector": "atorch_b200.utils.inspector",
    "atorch.kernels": "atorch_b200.ops",
    "atorch.ops.op_builder": "atorch_b200.ops.quantizer",
    "atorch.ops.quantizer": "atorch_b200.ops.quantizer",
    "atorch.data.shm_dataloader": "atorch_b200.data.shm_context",
    "atorch.data.elastic_dataloader": "atorch_b200.data.elastic_dataset",
    "atorch.data.unshuffled_batch_dataloader": "atorch_b200.data.unordered_dataloader",
}


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target):
        self.target = target

    def create_module(self, spec):
        return importlib.import_module(self.target)

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("atorch."):
            return None
        tgt = _RENAMES.get(fullname, "atorch_b200." + fullname[len("atorch."):])
        try:
            if importlib.util.find_spec(tgt) is None:
                return None
        except (ImportError, ValueError, AttributeError):
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(tgt))
        real = importlib.util.find_spec(tgt)
        if real is not None and real.submodule_search_locations is not None:
            spec.submodule_search_locations = list(real.submodule_search_locations)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

if not os.environ.get("ATORCH_DISABLE_ADDON"):
    try:
        importlib.import_module("atorch_addon")
    except ImportError:
        pass
