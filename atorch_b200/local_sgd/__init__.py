from .anomaly import OnlineDynamicEWMA
from .averager import (OuterOptimPeriodicModelAverager, PostLocalSGDState, StatefulPostLocalSGDOptimizer,
                       post_localSGD_hook)
from .configs import GTAConfig, LocalSGDConfig, OuterOptimizerConfig
from .reducers import GTAReducer, LinearReducer, TensorReducer, sparsify


def patch_local_sgd_to_fsdp():
    """Nothing to patch: the sharded engine implements local SGD natively (see ``local_sgd.sharded``)."""
    return True
