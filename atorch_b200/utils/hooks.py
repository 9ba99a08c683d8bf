"""Process-wide hook registry: callbacks the training loop calls for GPU-utilisation accounting, metric reports and
extra tensorboard scalars. (Reference: atorch/utils/hooks.py:5-30.)"""
from enum import auto
from typing import Callable, Dict, List


class ATorchHooks:
    COMPUTE_GPU_UTIL_HOOK = auto()
    REPORT_METRICS_HOOK = auto()
    ADDITIONAL_TENSORBOARD_HOOK = auto()

    hooks: Dict[object, List[Callable]] = {}

    @staticmethod
    def register_hook(hook_type, hook_func: Callable) -> None:
        """Idempotent per (type, function)."""
        funcs = ATorchHooks.hooks.setdefault(hook_type, [])
        if hook_func not in funcs:
            funcs.append(hook_func)

    @staticmethod
    def remove_hook(hook_type, hook_func: Callable) -> None:
        funcs = ATorchHooks.hooks.get(hook_type, [])
        if hook_func in funcs:
            funcs.remove(hook_func)

    @staticmethod
    def call_hooks(hook_type, *args, **kwargs) -> None:
        for func in list(ATorchHooks.hooks.get(hook_type, [])):
            func(*args, **kwargs)
