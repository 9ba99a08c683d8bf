from .gating import SwitchGate, TopkGate, TopNRouter, topk_gating
from .grouped_gemm_moe import Grouped_GEMM_MoE
from .moe_layer import Experts, MOELayer, get_experts_process_group, set_experts_process_group
from .token_dispatcher import MoEAllGatherTokenDispatcher, MoEAllToAllTokenDispatcher
from .ddp import (MoEMixtureDistributedDataParallel, get_experts_ddp_process_group,  # noqa: E402
                  set_experts_ddp_process_group)
