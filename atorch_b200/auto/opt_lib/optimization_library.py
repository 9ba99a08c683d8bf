"""Registry of optimisation methods, keyed by the names users write in ``load_strategy``.

(Reference: atorch/auto/opt_lib/optimization_library.py:23-81; the 17 method names are API.)
"""
from __future__ import annotations

from .amp import AmpNativeOptimization, HalfOptimization
from .checkpoint import CheckpointOptimization
from .misc import (DeepSpeed3DParallelOptimization, Fp8Optimization, MixedParallelOptimization,
                   NativeDynamoOptimization, PipelineParallelOptimization, SequenceParallelOptimization,
                   TensorParallelOptimization)
from .module_replace import ModuleReplaceOptimization
from .parallel_mode import AutoDDPOptimization, ParallelModeOptimization
from .zero import FSDP2Optimization, FSDPOptimization, Zero1Optimization, Zero2Optimization

SEMIAUTO_STRATEGIES = ("tensor_parallel", "mixed_parallel", "pipeline_parallel")


class OptimizationLibrary:
    def __init__(self):
        self.opts = {}
        self.group = {}
        for cls in (Zero1Optimization, Zero2Optimization, FSDPOptimization, FSDP2Optimization,
                    ParallelModeOptimization, AutoDDPOptimization, AmpNativeOptimization, Fp8Optimization,
                    TensorParallelOptimization, ModuleReplaceOptimization, CheckpointOptimization,
                    NativeDynamoOptimization, PipelineParallelOptimization, MixedParallelOptimization,
                    SequenceParallelOptimization, HalfOptimization, DeepSpeed3DParallelOptimization):
            self.register_opt(cls())

    def register_opt(self, opt) -> None:
        self.opts[opt.name] = opt
        self.group.setdefault(opt.group, []).append(opt.name)

    def __getitem__(self, name):
        return self.opts[name]

    def __contains__(self, name):
        return name in self.opts

    def validate_strategy(self, strategy):
        """(ok, names of unknown methods)."""
        bad = [o[0] for o in strategy if o[0] not in self.opts]
        return (len(bad) == 0, bad)
