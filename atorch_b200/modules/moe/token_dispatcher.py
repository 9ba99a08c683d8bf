"""Token dispatchers of the expert-parallel MoE: AllToAll (variable splits) and AllGather.

AllToAll: tokens are permuted by global expert id, split by owning rank, exchanged with one
all-to-all-v, regrouped by local expert; the combine path mirrors it and applies the routing
probabilities. Counts are exchanged with one small all-to-all on the device; the host reads the
split sizes once per layer (needed by the variable-size exchange of torch.distributed).
(Reference: atorch/modules/moe/token_dispatcher.py:89-1022.)
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

from ...communication.functions import (all_to_all, gather_from_expert_parallel_region_to_moe,
                                        reduce_scatter_to_expert_parallel_region_from_moe)
from ...ops import moe as moe_ops


class MoEAllToAllTokenDispatcher:
    def __init__(self, num_local_experts: int, local_expert_indices: List[int], num_experts: int, topk: int,
                 ep_group=None, use_expert_parallelism: bool = True):
        self.num_local_experts, self.local_expert_indices = num_local_experts, local_expert_indices
        self.num_experts, self.topk = num_experts, topk
        self.ep_group = ep_group
        self.ep_size = dist.get_world_size(ep_group) if (use_expert_parallelism and dist.is_initialized()) else 1

    def token_permutation(self, hidden_states, probs, indices, se_fn1: Optional[Callable] = None):
        self.hidden_shape = hidden_states.shape
        self.probs = probs
        x = hidden_states.reshape(-1, hidden_states.shape[-1])
        self.num_tokens = x.shape[0]
        counts = moe_ops.tokens_per_expert(indices, self.num_experts)             # [E] global ids
        permuted, self.sorted_idx = moe_ops.permute(x, indices)
        se_out = None
        if self.ep_size == 1:
            if se_fn1 is not None:
                se_out = se_fn1(hidden_states)
            self.tokens_per_local_expert = counts
            return permuted, counts, se_out
        ne = self.num_local_experts
        send_counts = counts.view(self.ep_size, ne)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=self.ep_group)
        host = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()           # the one host sync
        self.input_splits, self.output_splits = host[0].tolist(), host[1].tolist()
        recv = all_to_all(self.ep_group, permuted, self.output_splits, self.input_splits)
        if se_fn1 is not None:
            se_out = se_fn1(hidden_states)
        self.recv_counts = recv_counts                                             # [ep, ne]: from rank r for local e
        if ne > 1:
            # rows arrive grouped by source rank, then by local expert: regroup by local expert
            src_expert = torch.repeat_interleave(
                torch.arange(ne, device=x.device).repeat(self.ep_size), recv_counts.reshape(-1))
            self.local_sort = torch.argsort(src_expert, stable=True)
            recv = recv.index_select(0, self.local_sort)
        else:
            self.local_sort = None
        tokens_local = recv_counts.sum(0)
        return recv, tokens_local, se_out

    def token_unpermutation(self, expert_output, se_fn2: Optional[Callable] = None, se_fn2_additional_input=None):
        se_out = None
        if self.ep_size > 1:
            if self.local_sort is not None:
                inv = torch.empty_like(self.local_sort)
                inv[self.local_sort] = torch.arange(self.local_sort.numel(), device=inv.device)
                expert_output = expert_output.index_select(0, inv)
            expert_output = all_to_all(self.ep_group, expert_output, self.input_splits, self.output_splits)
        if se_fn2 is not None:
            se_out = se_fn2(*se_fn2_additional_input) if isinstance(se_fn2_additional_input, (tuple, list)) \
                else se_fn2(se_fn2_additional_input)
        out = moe_ops.unpermute(expert_output, self.sorted_idx, self.probs, self.topk, self.num_tokens)
        return out.view(self.hidden_shape), se_out


class MoEAllGatherTokenDispatcher:
    """Every rank gathers all tokens, keeps those routed to its local experts; outputs are
    reduce-scattered back (suits small expert-parallel groups)."""

    def __init__(self, num_local_experts: int, local_expert_indices: List[int], num_experts: int, topk: int,
                 ep_group=None, use_expert_parallelism: bool = True):
        self.num_local_experts, self.local_expert_indices = num_local_experts, local_expert_indices
        self.num_experts, self.topk, self.ep_group = num_experts, topk, ep_group
        self.ep_size = dist.get_world_size(ep_group) if (use_expert_parallelism and dist.is_initialized()) else 1

    def token_permutation(self, hidden_states, probs, indices, se_fn1=None):
        self.hidden_shape = hidden_states.shape
        x = hidden_states.reshape(-1, hidden_states.shape[-1])
        if self.ep_size > 1:
            x = gather_from_expert_parallel_region_to_moe(x, self.ep_group)
            probs = gather_from_expert_parallel_region_to_moe(probs.contiguous(), self.ep_group)
            indices = gather_from_expert_parallel_region_to_moe(indices.contiguous(), self.ep_group)
        se_out = se_fn1(hidden_states) if se_fn1 is not None else None
        lo, hi = self.local_expert_indices[0], self.local_expert_indices[-1]
        flat_idx, flat_p = indices.reshape(-1), probs.reshape(-1)
        mine = (flat_idx >= lo) & (flat_idx <= hi)
        self.slot = torch.nonzero(mine, as_tuple=False)[:, 0]                      # positions in [T*k]
        local_e = flat_idx[self.slot] - lo
        order = torch.argsort(local_e, stable=True)
        self.slot = self.slot[order]
        self.local_probs = flat_p[self.slot]
        self.total_tokens = x.shape[0]
        tokens_local = torch.bincount(local_e, minlength=self.num_local_experts)
        return x.index_select(0, self.slot // self.topk), tokens_local, se_out

    def token_unpermutation(self, expert_output, se_fn2=None, se_fn2_additional_input=None):
        weighted = expert_output * self.local_probs.unsqueeze(-1).to(expert_output.dtype)
        out = torch.zeros(self.total_tokens, expert_output.shape[-1], dtype=expert_output.dtype,
                          device=expert_output.device)
        out = out.index_add(0, self.slot // self.topk, weighted)
        if self.ep_size > 1:
            out = reduce_scatter_to_expert_parallel_region_from_moe(out, self.ep_group)
        se_out = None
        if se_fn2 is not None:
            se_out = se_fn2(*se_fn2_additional_input) if isinstance(se_fn2_additional_input, (tuple, list)) \
                else se_fn2(se_fn2_additional_input)
        return out.view(self.hidden_shape), se_out
