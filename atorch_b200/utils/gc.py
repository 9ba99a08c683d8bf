"""Manual garbage collection: Python's cyclic collector is switched off and run explicitly every N steps, on
all ranks at the same step, so that a collection pause never lands on one rank in the middle of a collective.
(Reference: ``ManualGarbageCollection`` in atorch/utils/gc.py.)"""
from __future__ import annotations

import gc


class ManualGarbageCollection:
    def __init__(self, gc_freq: int = 1000, disable_auto_gc: bool = True):
        assert gc_freq > 0, "gc_freq must be a positive integer"
        self.gc_freq = gc_freq
        self.collections = 0
        if disable_auto_gc:
            gc.disable()
        gc.collect(1)

    def run(self, step_count: int) -> bool:
        if step_count > 1 and step_count % self.gc_freq == 0:
            gc.collect(1)
            self.collections += 1
            return True
        return False

    @staticmethod
    def restore() -> None:
        gc.enable()
