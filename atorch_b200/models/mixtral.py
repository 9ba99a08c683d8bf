"""Mixtral-style sparse mixture-of-experts decoder: Llama attention (grouped-query) + a top-k routed expert
MLP per layer (``TopNRouter`` + ``Grouped_GEMM_MoE``), optionally with block-scaled fp8 expert GEMMs and
expert parallelism over the ``expert`` group.

Config of the MoE benchmark: 16 layers, hidden 4096, 32 query / 8 KV heads, 8 experts, top-2, expert FFN
14336, vocab 32000. (Reference: examples/moe/moe_modules.py:57-112 router + ``_SparseMLP``,
atorch/modules/moe/grouped_gemm_moe.py:349.)"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..modules.moe import Grouped_GEMM_MoE, TopNRouter
from ..utils.checkpoint import checkpoint_module
from .llama import LlamaConfig, RMSNorm, causal_lm_loss


@dataclass
class MixtralConfig(LlamaConfig):
    num_experts: int = 8
    top_k: int = 2
    expert_intermediate_size: int = 14336
    use_expert_parallelism: bool = False
    fp8_experts: bool = False
    router_aux_loss_coef: float = 0.01
    router_z_loss_coef: float = 0.0
    token_dispatcher_type: str = "AllToAll"     # "PeerMemory": capacity routing over NVLink peer memory
    capacity_factor: float = 1.25                # slots per (rank, expert) = factor * tokens * top_k / experts

    @staticmethod
    def mixtral_bench(**kw) -> "MixtralConfig":
        d = dict(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=16,
                 num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=4096, num_experts=8, top_k=2,
                 expert_intermediate_size=14336)
        d.update(kw)
        return MixtralConfig(**d)

    @staticmethod
    def tiny_moe(**kw) -> "MixtralConfig":
        d = dict(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                 num_key_value_heads=1, max_position_embeddings=64, num_experts=4, top_k=2,
                 expert_intermediate_size=128)
        d.update(kw)
        return MixtralConfig(**d)


class SparseMLP(nn.Module):
    def __init__(self, cfg: MixtralConfig):
        super().__init__()
        self.router = TopNRouter(cfg.hidden_size, cfg.num_experts, cfg.top_k, aux_loss_coef=cfg.router_aux_loss_coef,
                                 z_loss_coef=cfg.router_z_loss_coef)
        self.experts = Grouped_GEMM_MoE(cfg.hidden_size, cfg.expert_intermediate_size, 0.0, cfg.num_experts, cfg.top_k,
                                        use_swiglu=True, use_expert_parallelism=cfg.use_expert_parallelism,
                                        implementation_type="Megatron", token_dispatcher_type=cfg.token_dispatcher_type,
                                        fp8=cfg.fp8_experts, initializer_range=cfg.initializer_range,
                                        capacity_factor=cfg.capacity_factor)

    def forward(self, x):
        probs, idx = self.router(x)
        return self.experts(x, probs, idx)


class MixtralDecoderLayer(nn.Module):
    _atb_direct_grad_params = ("qkv_proj.weight", "o_proj.weight", "input_layernorm.weight",
                               "post_attention_layernorm.weight")

    def __init__(self, cfg: MixtralConfig, layer_idx: int = 0):
        super().__init__()
        self.config = cfg
        h, d = cfg.hidden_size, cfg.head_dim
        self.n_q, self.n_kv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.input_layernorm = RMSNorm(h, cfg.rms_norm_eps)
        self.qkv_proj = nn.Linear(h, (self.n_q + 2 * self.n_kv) * d, bias=False)
        self.o_proj = nn.Linear(self.n_q * d, h, bias=False)
        self.post_attention_layernorm = RMSNorm(h, cfg.rms_norm_eps)
        self.block_sparse_moe = SparseMLP(cfg)

    def forward(self, h, cos, sin, positions=None, attn_kwargs=None):
        B, S, _ = h.shape
        d = self.config.head_dim
        x = self.input_layernorm(h)
        qkv = ops.rope(ops.linear(x, self.qkv_proj.weight), cos, sin, self.n_q + self.n_kv, d, positions)
        qkv = qkv.view(B, S, self.n_q + 2 * self.n_kv, d)
        a = ops.attention(qkv[:, :, : self.n_q], qkv[:, :, self.n_q: self.n_q + self.n_kv],
                          qkv[:, :, self.n_q + self.n_kv:], **(attn_kwargs or {"causal": True}))
        h = ops.linear(a.reshape(B, S, self.n_q * d), self.o_proj.weight, residual=h)
        return h + self.block_sparse_moe(self.post_attention_layernorm(h))


class MixtralModel(nn.Module):
    def __init__(self, config: MixtralConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([MixtralDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self._atb_direct_grad_params = ("norm.weight", "lm_head.weight")
        self._rope = {}
        self.apply(self._init_weights)

    def _init_weights(self, m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=self.config.initializer_range)

    def aux_loss(self):
        tot = 0.0
        for l in self.layers:
            r = l.block_sparse_moe.router
            for v in (r.aux_loss, r.z_loss):
                if v is not None:
                    tot = tot + v
        return tot

    def forward(self, input_ids, labels=None, return_logits: bool = True):
        B, S = input_ids.shape
        key = (S, str(input_ids.device))
        if key not in self._rope:
            self._rope = {key: ops.rope_tables(S, self.config.head_dim, self.config.rope_theta, input_ids.device)}
        cos, sin = self._rope[key]
        h = self.embed_tokens(input_ids)
        for layer in self.layers:
            if self.config.gradient_checkpointing and self.training and torch.is_grad_enabled():
                h = checkpoint_module(layer, h, cos, sin)
            else:
                h = layer(h, cos, sin)
        logits = ops.linear(self.norm(h), self.lm_head.weight)
        loss = None
        if labels is not None:
            loss = causal_lm_loss(logits, labels) + self.aux_loss()
        return (loss, logits if return_logits else None)
