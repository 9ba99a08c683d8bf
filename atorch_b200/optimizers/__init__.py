from .adaml import AdamL
from .agd import AGD
from .bf16_optimizer import BF16Optimizer
from .wsam import WeightedSAM
from .adam_offload import PartitionAdam
