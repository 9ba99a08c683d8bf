"""atorch_b200: a Blackwell-native (sm_100a) hybrid-parallel training framework with the
capabilities and public API of ATorch.

Layers: ``csrc`` (CUDA kernels) -> ``ops`` (autograd operators) -> ``modules`` / ``models`` /
``optimizers`` -> ``parallel`` (sharded data parallel, DDP, tensor / pipeline / sequence / expert
parallel, local SGD) -> ``auto`` (``auto_accelerate`` and strategies) -> ``trainer``; ``distributed``
is the process-group runtime under all of them.
"""
from .distributed.distributed import (coworker_size, init_distributed, local_rank, rank, reset_distributed,
                                      world_size)

__version__ = "0.1.0"
