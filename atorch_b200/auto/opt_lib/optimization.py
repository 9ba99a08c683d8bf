"""Base class of optimisation methods.

A method has a ``name`` (the string users write in ``load_strategy``), a ``group`` (methods of one
group exclude each other in the automatic search) and three hooks:

* ``tune(model_context, config, strategy, apply_transform, time_limit)`` -> ``(ok, best_config, ctx)``
* ``transform(model_context, config)`` registers wrappers on the context (cheap, no side effects)
* ``apply_wrapper(model_context, wrapper_name, wrapper_config)`` does the actual work

(Reference interface: atorch/auto/opt_lib/optimization.py:25-78.)
"""
from __future__ import annotations


class Optimization:
    def __init__(self, name: str, group: str, is_tunable: bool, is_distributed: bool = False):
        self.name, self.group, self.is_tunable, self.is_distributed = name, group, is_tunable, is_distributed

    def distributed_only(self, config=None) -> bool:
        return self.is_distributed

    def device_supported(self, config=None, device_capability=None) -> bool:
        return True

    def tune(self, model_context, config=None, strategy=None, apply_transform: bool = True, time_limit=None):
        if apply_transform:
            model_context = self.transform(model_context, config)
        return True, config, model_context

    def transform(self, model_context, config=None):
        return model_context

    @staticmethod
    def apply_wrapper(model_context, wrapper_name, wrapper_config=None):
        return model_context

    @staticmethod
    def reset(config):
        pass
