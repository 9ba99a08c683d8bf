"""``Grouped_GEMM_MoE``: expert MLPs as grouped GEMMs with expert parallelism.

``forward(hidden_states, expert_weights, top_experts, se_fn1, se_fn2, se_fn2_additional_input)``:
``expert_weights`` / ``top_experts`` are the router's ``[tokens, topk]`` probabilities and expert ids.
Tokens are dispatched to the ranks owning their experts, run through ``w1`` (merged gate|up when
``use_swiglu`` and ``merge_w1_v1``) -> activation -> ``w2`` with one grouped GEMM each, and combined
with the routing probabilities. Weights: ``w1 [E_local, F(*2), H]`` (``transpose_w1``) or
``[E_local, H, F(*2)]``, ``w2 [E_local, F, H]``, optional ``v1``. ``se_fn1`` / ``se_fn2`` run a shared
expert while the exchanges are in flight. With ``fp8=True`` the expert GEMMs run on the block-scaled
fp8 path (activations 1x128, weights 128x128 scales).
(Reference: atorch/modules/moe/grouped_gemm_moe.py:349-901.)
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn

from ... import ops
from ...distributed import distributed as D
from ...ops import moe as moe_ops
from .token_dispatcher import MoEAllGatherTokenDispatcher, MoEAllToAllTokenDispatcher


class _ScaleGradient(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return x

    @staticmethod
    def backward(ctx, g):
        return g * ctx.scale, None


class Grouped_GEMM_MoE(nn.Module):
    def __init__(self, hidden_size, expert_intermediate_size, output_dropout_prob, num_experts, topk,
                 use_swiglu=False, use_bias=False, initializer_range=0.02, use_expert_parallelism=False,
                 expert_parallel_group=None, merge_w1_v1=True, transpose_w1=True, is_scale_gradient=False,
                 implementation_type="Megatron", token_dispatcher_type="AllToAll", fp8: bool = False,
                 capacity_factor: float = 1.25):
        super().__init__()
        self.hidden_size, self.expert_intermediate_size = hidden_size, expert_intermediate_size
        self.num_experts, self.topk, self.use_swiglu, self.use_bias = num_experts, topk, use_swiglu, use_bias
        self.merge_w1_v1, self.transpose_w1, self.fp8 = merge_w1_v1, transpose_w1, fp8
        self.use_expert_parallelism = use_expert_parallelism
        self.expert_parallel_group = None
        ep = 1
        if use_expert_parallelism:
            self.expert_parallel_group = expert_parallel_group if expert_parallel_group is not None \
                else D.parallel_group("expert")
            ep = dist.get_world_size(self.expert_parallel_group) if dist.is_initialized() else 1
        assert num_experts % ep == 0
        self.num_local_experts = num_experts // ep
        self.gradient_scale = (1.0 / ep) if (use_expert_parallelism and is_scale_gradient) else None
        E, F, H = self.num_local_experts, expert_intermediate_size, hidden_size
        f1 = F * (2 if (use_swiglu and merge_w1_v1) else 1)
        self.w1 = nn.Parameter(torch.empty((E, f1, H) if transpose_w1 else (E, H, f1)))
        self.w2 = nn.Parameter(torch.empty(E, F, H))
        if use_swiglu and not merge_w1_v1:
            self.v1 = nn.Parameter(torch.empty((E, F, H) if transpose_w1 else (E, H, F)))
        else:
            self.v1 = None
        if use_bias:
            self.b1 = nn.Parameter(torch.zeros(E, f1))
            self.b2 = nn.Parameter(torch.zeros(E, H))
        self.dropout = nn.Dropout(output_dropout_prob)
        for w in (self.w1, self.w2, self.v1):
            if w is not None:
                nn.init.normal_(w, mean=0.0, std=initializer_range)
        rank = (dist.get_rank(self.expert_parallel_group) if (use_expert_parallelism and dist.is_initialized())
                else 0)
        local = [rank * E + i for i in range(E)]
        self.peer_exchange = False
        if token_dispatcher_type == "PeerMemory":
            # capacity-factor routing with the exchange done by this package's kernels over NVLink peer
            # memory (csrc/moe.cu); needs expert parallelism on 2..8 GPUs of one NVSwitch domain
            from .peer_dispatch import MoEPeerMemoryTokenDispatcher, available

            if use_expert_parallelism and available(self.expert_parallel_group):
                self.token_dispatcher = MoEPeerMemoryTokenDispatcher(
                    E, local, num_experts, topk, self.expert_parallel_group, True, capacity_factor)
                self.peer_exchange = True
                return
            token_dispatcher_type = "AllToAll"
        cls = MoEAllGatherTokenDispatcher if token_dispatcher_type in ("AllGather", "MindSpeedAllGather") \
            else MoEAllToAllTokenDispatcher
        self.token_dispatcher = cls(E, local, num_experts, topk, self.expert_parallel_group, use_expert_parallelism)

    def has_v1(self) -> bool:
        return self.v1 is not None

    def _scaled(self, w):
        return w if self.gradient_scale is None else _ScaleGradient.apply(w, self.gradient_scale)

    def _gmm(self, x, w, sizes, w_is_nk: bool):
        """x[g] @ W[g]^T when ``w_is_nk`` ([E, N, K]) else x[g] @ W[g] ([E, K, N])."""
        if self.fp8:
            from ..fp8.grouped import grouped_scaled_linear

            return grouped_scaled_linear(x, w if w_is_nk else w.transpose(1, 2), sizes)
        return moe_ops.grouped_gemm(x, w, sizes, trans_b=w_is_nk)

    def compute_expert_slots(self, x: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        """Expert MLP over an expert buffer ``[E_local * W * capacity, H]`` whose groups of ``capacity`` slots
        are filled up to ``counts`` (int32, on the device) and zero beyond: grouped GEMMs that skip empty
        tiles, no host sync. With fp8 experts the block-scaled path runs over all slots (static shapes)."""
        from .peer_dispatch import grouped_linear

        d = self.token_dispatcher
        cap, W = d.bufs.capacity, d.ep_size
        w1, w2 = self._scaled(self.w1), self._scaled(self.w2)
        if self.fp8:
            sizes = [W * cap] * self.num_local_experts
            lin1 = lambda t, w, nk: self._gmm(t, w, sizes, nk)
        else:
            lin1 = lambda t, w, nk: grouped_linear(t, w, counts, cap, W, nk)
        h = lin1(x, w1, self.transpose_w1)
        if self.use_swiglu:
            h = torch.nn.functional.silu(h) * lin1(x, self._scaled(self.v1), self.transpose_w1) \
                if self.v1 is not None else ops.swiglu(h)
        else:
            h = torch.nn.functional.gelu(h)
        return lin1(h, w2, False)

    def compute_expert(self, x: torch.Tensor, tokens_per_expert: torch.Tensor) -> torch.Tensor:
        if self.peer_exchange:
            return self.compute_expert_slots(x, tokens_per_expert)
        sizes = tokens_per_expert.tolist()
        w1, w2 = self._scaled(self.w1), self._scaled(self.w2)
        h = self._gmm(x, w1, sizes, self.transpose_w1)
        if self.use_bias:
            eidx = torch.repeat_interleave(torch.arange(len(sizes), device=x.device), tokens_per_expert)
            h = ops.bias_gather_add(h, self.b1.to(h.dtype), eidx)
        if self.use_swiglu:
            if self.v1 is not None:
                up = self._gmm(x, self._scaled(self.v1), sizes, self.transpose_w1)
                h = torch.nn.functional.silu(h) * up
            else:
                h = ops.swiglu(h)
        else:
            h = torch.nn.functional.gelu(h)
        out = self._gmm(h, w2, sizes, False)
        if self.use_bias:
            out = ops.bias_gather_add(out, self.b2.to(out.dtype), eidx)
        return out

    def forward(self, hidden_states, expert_weights, top_experts, se_fn1: Optional[Callable] = None,
                se_fn2: Optional[Callable] = None, se_fn2_additional_input=None):
        expert_weights = expert_weights.view(-1, expert_weights.shape[-1])
        top_experts = top_experts.view(-1, top_experts.shape[-1])
        x, tokens_local, se_mid = self.token_dispatcher.token_permutation(hidden_states, expert_weights, top_experts,
                                                                         se_fn1)
        y = self.compute_expert(x, tokens_local)
        extra = se_fn2_additional_input if se_fn2_additional_input is not None else se_mid
        out, se_out = self.token_dispatcher.token_unpermutation(y, se_fn2, extra)
        out = self.dropout(out)
        if se_fn2 is not None and se_out is not None:
            out = out + se_out
        elif se_fn1 is not None and se_fn2 is None and se_mid is not None:
            out = out + se_mid
        return out
