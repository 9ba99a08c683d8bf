from .accelerate import AutoAccelerateResult, auto_accelerate, get_strategy, save_strategy
from .strategy import Strategy
