from .gating import SwitchGate, TopkGate, TopNRouter, topk_gating
from .grouped_gemm_moe import Grouped_GEMM_MoE
from .moe_layer import Experts, MOELayer, get_experts_process_group, set_experts_process_group
from .token_dispatcher import MoEAllGatherTokenDispatcher, MoEAllToAllTokenDispatcher
