"""(Reference: atorch/utils/dev_utils.py:1-10.)"""
import functools


def raise_not_impl(func):
    """Decorator for interface methods: calling one raises ``NotImplementedError`` naming the concrete class."""

    @functools.wraps(func)
    def wrapper(self, *args, **kwargs):
        raise NotImplementedError(f"{type(self).__name__} does not implement function {func.__name__}")

    return wrapper
