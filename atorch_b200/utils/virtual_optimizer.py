"""Memory estimation without allocating: per-rank bytes of parameters, gradients and optimizer state for a
given layout (data/tensor/pipeline sizes, sharded optimizer or not), used to reject infeasible plans early.
(Reference: atorch/utils/virtual_optimizer/ which emulates Megatron's optimizer allocation.)"""
from __future__ import annotations

from typing import Dict

import torch.nn as nn


def estimate_training_memory(model: nn.Module, data: int = 1, tensor: int = 1, pipe: int = 1,
                             shard_params: bool = True, shard_optimizer: bool = True, param_bytes: int = 2,
                             grad_bytes: int = 4, state_bytes: int = 12) -> Dict[str, float]:
    n = sum(p.numel() for p in model.parameters()) / (tensor * pipe)
    params = n * param_bytes / (data if shard_params else 1)
    grads = n * grad_bytes / (data if shard_params else 1)
    state = n * state_bytes / (data if shard_optimizer else 1)
    return {"params": params, "grads": grads, "optimizer_state": state, "total": params + grads + state}
