"""Configuration dataclasses of local SGD / EDiT (same fields as atorch/local_sgd/configs/configs.py:10-49)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Type

from torch.optim import Optimizer


@dataclass
class LocalSGDConfig:
    use_async: bool = False                 # True: replicas sync by wall-clock time instead of step count
    local_sgd_sync_interval: int = 1        # H: inner steps between two outer steps
    local_sgd_sync_time: float = 600.0      # async mode: seconds between outer steps
    min_total_global_steps: int = 100
    use_step_weight: bool = False
    step_weight_ratio: float = 0.5
    local_sgd_warmup_steps: int = 0         # fully synchronous steps before local SGD starts
    gradient_accumulation_steps: int = 1
    clip_pseudo_grad: Optional[float] = None
    pseudo_gradnorm_reduce: bool = False
    weight_softmax_temperature: Optional[float] = None
    skip_anomaly: bool = False
    ewma_alpha: float = 0.02
    ewma_warmup_steps: int = 120
    ewma_threshold: int = 3
    cpu_offload: bool = False
    is_debug: bool = False


@dataclass
class OuterOptimizerConfig:
    outer_optim_class: Optional[Type[Optimizer]] = None
    outer_optim_kwargs: dict = field(default_factory=dict)


@dataclass
class GTAConfig:
    reducer: Optional[str] = None                  # "linear" | "gta"
    consensus_method: Optional[str] = None         # "sum" | "count"
    sparsification_method: Optional[str] = None    # "magnitude" | "random" | "rescaled_random"
    normalize: bool = True
    density: float = 1.0
    int8_mask: bool = False
