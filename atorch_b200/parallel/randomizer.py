"""RNG streams for model-parallel training: one generator state per set of "same" groups.

``get_randomizer("tensor")`` yields an RNG whose draws are identical on all ranks of the tensor
group (seed independent of the tensor rank) and differ across the other dims; ``get_randomizer()``
differs on every rank. ``with randomizer.fork():`` swaps the CPU and CUDA generator states in and
out, like Megatron's RNG tracker.
(Reference: atorch/modules/distributed_modules/randomizer.py:9-142.)
"""
from __future__ import annotations

import contextlib
import zlib
from typing import Dict, Tuple

import torch

from ..distributed import distributed as D

_BASE_SEED = 1234
_RANDOMIZERS: Dict[Tuple[str, ...], "MultiDimParallelRandomizer"] = {}


def init_randomizer(base_seed: int = 1234) -> None:
    global _BASE_SEED
    _BASE_SEED = base_seed
    _RANDOMIZERS.clear()


class MultiDimParallelRandomizer:
    def __init__(self, *same_groups: str, base_seed=None):
        self.same_groups = tuple(same_groups)
        seed = _BASE_SEED if base_seed is None else base_seed
        cfg = D.parallel_config()
        offset, stride = 0, 1
        if cfg is not None:
            for name, size in cfg[0]:
                if name not in self.same_groups:
                    offset += (D.parallel_rank(name) or 0) * stride
                    stride *= size
        elif not self.same_groups:
            offset = D.rank() or 0
        # crc32, not hash(): Python salts string hashes per process, and ranks must agree on the seed
        self.seed = seed + 2718 * (zlib.crc32(",".join(self.same_groups).encode()) % 1000) + offset
        self.cpu_state = torch.Generator().manual_seed(self.seed).get_state()
        self.cuda_state = None

    @contextlib.contextmanager
    def fork(self):
        cpu_now = torch.get_rng_state()
        torch.set_rng_state(self.cpu_state)
        use_cuda = torch.cuda.is_available() and torch.cuda.is_initialized()
        if use_cuda:
            cuda_now = torch.cuda.get_rng_state()
            if self.cuda_state is None:
                torch.cuda.manual_seed(self.seed)
            else:
                torch.cuda.set_rng_state(self.cuda_state)
        try:
            yield
        finally:
            self.cpu_state = torch.get_rng_state()
            torch.set_rng_state(cpu_now)
            if use_cuda:
                self.cuda_state = torch.cuda.get_rng_state()
                torch.cuda.set_rng_state(cuda_now)


def get_randomizer(*same_groups: str) -> MultiDimParallelRandomizer:
    key = tuple(same_groups)
    if key not in _RANDOMIZERS:
        _RANDOMIZERS[key] = MultiDimParallelRandomizer(*same_groups)
    return _RANDOMIZERS[key]


def get_MDPRInstance() -> MultiDimParallelRandomizer:
    """The stream that differs on every rank (the name the original package uses for its default instance)."""
    return get_randomizer()
