"""Class-level registry of per-``auto_accelerate``-call state (half dtype, grad scaler, ...).

Each ``auto_accelerate`` call bumps ``counter``; attributes are dicts keyed by that counter.
(Reference: atorch/auto/auto_accelerate_context.py:4-31.)
"""


class AutoAccelerateContext:
    counter = 0

    @classmethod
    def add_ac_attr(cls, name, value):
        if not hasattr(cls, name):
            setattr(cls, name, value)

    @classmethod
    def get(cls, name, default=None):
        d = getattr(cls, name, None)
        return default if d is None else d.get(cls.counter, default)

    @classmethod
    def set(cls, name, value):
        if not hasattr(cls, name):
            setattr(cls, name, {})
        getattr(cls, name)[cls.counter] = value

    @classmethod
    def reset(cls):
        for k in [k for k, v in vars(cls).items() if not k.startswith("__") and isinstance(v, dict)]:
            delattr(cls, k)
        cls.counter = 0
