"""(Reference: atorch/optimizers/utils.py:23-27.)"""
import contextlib


def whether_to_sync(model, sync: bool = False):
    """Context for one of several backward passes of a step (sharpness-aware optimizers run two): gradient
    synchronisation of a data-parallel wrapper is suppressed unless ``sync``."""
    if not sync and hasattr(model, "no_sync"):
        return model.no_sync()
    return contextlib.ExitStack()
