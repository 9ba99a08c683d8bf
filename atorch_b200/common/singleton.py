"""(Reference: atorch/common/singleton.py:4-25.)"""
from typing import Dict


class SingletonMeta(type):
    """Metaclass: the first call constructs the one instance of a class, later calls return it and must not pass
    arguments (they would be ignored silently otherwise)."""

    _instances: Dict[type, object] = {}

    def __call__(cls, *args, **kwargs):
        inst = SingletonMeta._instances.get(cls)
        if inst is None:
            inst = SingletonMeta._instances[cls] = super().__call__(*args, **kwargs)
        else:
            assert not args and not kwargs, f"{cls.__name__} is a singleton class and a instance has been created."
        return inst
