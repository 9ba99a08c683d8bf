from .optimization import Optimization
from .optimization_library import SEMIAUTO_STRATEGIES, OptimizationLibrary
