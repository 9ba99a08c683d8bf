"""Megatron-style tensor-parallel transformer blocks on top of ``ColumnParallelLinear`` / ``RowParallelLinear``.

* ``ParallelSelfAttention``: fused q/k/v column-parallel projection (heads split over the group, grouped-query
  heads supported), attention on the local heads through ``ops.attention`` (flash kernels on a B200), attention
  dropout drawn from the rank-private RNG stream, row-parallel output projection.
* ``ParallelMLP``: column-parallel up (or fused gate/up for SwiGLU) and row-parallel down projection.
* ``ParallelTransformerLayer``: pre- or post-LayerNorm block (``apply_residual_connection_post_layernorm``);
  hidden dropout drawn from the stream shared by the tensor group (every rank holds the full hidden state and
  must drop the same elements). With ``sequence_parallel`` the hidden state between the blocks is split along
  the sequence and the linears use the fused all-gather→GEMM / GEMM→reduce-scatter kernels.
* ``from_unsharded``: builds a parallel block from an unsharded block description (the HF GPT-2, BERT and Llama
  layers have adapters below) by slicing its weights, and ``tp_checkpoint`` is activation checkpointing that
  replays both RNG streams in the recomputation.

One generic block replaces the per-architecture classes of the reference (MegatronBertAttention, CLIP, GLM,
GPT-NeoX ...: atorch/modules/distributed_modules/transformer.py:45-1801, activation_checkpointing.py:81-366).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...parallel.randomizer import get_randomizer
from .layers import ColumnParallelLinear, RowParallelLinear, _group, _ws


def _linear_from(weight: torch.Tensor, bias: Optional[torch.Tensor]) -> nn.Linear:
    lin = nn.Linear(weight.shape[1], weight.shape[0], bias=bias is not None, dtype=weight.dtype, device=weight.device)
    with torch.no_grad():
        lin.weight.copy_(weight)
        if bias is not None:
            lin.bias.copy_(bias)
    return lin


class ParallelSelfAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: Optional[int] = None, bias: bool = True,
                 causal: bool = True, attention_dropout: float = 0.0, process_group="tensor",
                 sequence_parallel: bool = False, qkv: Optional[nn.Linear] = None, out: Optional[nn.Linear] = None,
                 rotary: Optional[Callable] = None, dtype=None, device=None):
        super().__init__()
        self.group = _group(process_group)
        self.tp = _ws(self.group)
        kv = num_kv_heads or num_heads
        assert num_heads % self.tp == 0 and kv % self.tp == 0, "heads must divide by the tensor-parallel size"
        self.head_dim = hidden_size // num_heads
        self.heads, self.kv_heads = num_heads // self.tp, kv // self.tp
        self.causal, self.p_drop, self.rotary = causal, attention_dropout, rotary
        self.seq_par = sequence_parallel
        q_out, kv_out = num_heads * self.head_dim, kv * self.head_dim
        # q, k and v are three column-parallel projections stored separately so that grouped-query shapes
        # (q wider than k / v) slice cleanly
        split = (lambda lo, hi: _linear_from(qkv.weight[lo:hi], None if qkv.bias is None else qkv.bias[lo:hi])) \
            if qkv is not None else (lambda lo, hi: None)
        mk = lambda o, src: ColumnParallelLinear(hidden_size, o, bias, orig_module=src, process_group=process_group,  # noqa: E731
                                                 sequence_parallel=sequence_parallel, dtype=dtype, device=device)
        self.q_proj = mk(q_out, split(0, q_out))
        self.k_proj = mk(kv_out, split(q_out, q_out + kv_out))
        self.v_proj = mk(kv_out, split(q_out + kv_out, q_out + 2 * kv_out))
        self.out_proj = RowParallelLinear(q_out, hidden_size, bias, orig_module=out, process_group=process_group,
                                          sequence_parallel=sequence_parallel, dtype=dtype, device=device)

    def forward(self, x, key_padding_mask=None, position_ids=None):
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        B, S = q.shape[0], q.shape[1]
        q = q.view(B, S, self.heads, self.head_dim)
        k = k.view(B, S, self.kv_heads, self.head_dim)
        v = v.view(B, S, self.kv_heads, self.head_dim)
        if self.rotary is not None:
            q, k = self.rotary(q, k, position_ids)
        if self.p_drop > 0.0 and self.training:
            with get_randomizer().fork():            # different heads on every rank: private stream
                o = ops.attention(q, k, v, causal=self.causal, key_padding_mask=key_padding_mask, dropout_p=self.p_drop)
        else:
            o = ops.attention(q, k, v, causal=self.causal, key_padding_mask=key_padding_mask)
        return self.out_proj(o.reshape(B, S, self.heads * self.head_dim))


class ParallelMLP(nn.Module):
    def __init__(self, hidden_size: int, ffn_hidden_size: int, activation: str = "gelu", bias: bool = True,
                 process_group="tensor", sequence_parallel: bool = False, up: Optional[nn.Linear] = None,
                 gate: Optional[nn.Linear] = None, down: Optional[nn.Linear] = None, dtype=None, device=None):
        super().__init__()
        assert activation in ("gelu", "gelu_new", "relu", "swiglu")
        self.activation = activation
        mk = lambda src: ColumnParallelLinear(hidden_size, ffn_hidden_size, bias, orig_module=src,  # noqa: E731
                                              process_group=process_group, sequence_parallel=sequence_parallel,
                                              dtype=dtype, device=device)
        self.up_proj = mk(up)
        self.gate_proj = mk(gate) if activation == "swiglu" else None
        self.down_proj = RowParallelLinear(ffn_hidden_size, hidden_size, bias, orig_module=down,
                                           process_group=process_group, sequence_parallel=sequence_parallel,
                                           dtype=dtype, device=device)

    def forward(self, x):
        u = self.up_proj(x)
        if self.activation == "swiglu":
            u = F.silu(self.gate_proj(x)) * u
        elif self.activation == "relu":
            u = F.relu(u)
        else:
            u = F.gelu(u, approximate="tanh" if self.activation == "gelu_new" else "none")
        return self.down_proj(u)


@dataclass
class BlockSpec:
    """An unsharded transformer layer in the terms the parallel block needs (weights as ``nn.Linear``)."""
    hidden_size: int
    num_heads: int
    ffn_hidden_size: int
    qkv: nn.Linear
    attn_out: nn.Linear
    mlp_up: nn.Linear
    mlp_down: nn.Linear
    norm1: nn.Module
    norm2: nn.Module
    mlp_gate: Optional[nn.Linear] = None
    num_kv_heads: Optional[int] = None
    activation: str = "gelu"
    causal: bool = True
    post_layernorm: bool = False           # BERT: x = LN(x + f(x))
    attention_dropout: float = 0.0
    hidden_dropout: float = 0.0
    rotary: Optional[Callable] = None


class ParallelTransformerLayer(nn.Module):
    def __init__(self, spec: BlockSpec, process_group="tensor", sequence_parallel: bool = False):
        super().__init__()
        bias = spec.qkv.bias is not None
        self.post_ln, self.p_drop, self.seq_par = spec.post_layernorm, spec.hidden_dropout, sequence_parallel
        self.input_layernorm, self.post_attention_layernorm = spec.norm1, spec.norm2
        self.attention = ParallelSelfAttention(spec.hidden_size, spec.num_heads, spec.num_kv_heads, bias, spec.causal,
                                               spec.attention_dropout, process_group, sequence_parallel, spec.qkv,
                                               spec.attn_out, spec.rotary)
        self.mlp = ParallelMLP(spec.hidden_size, spec.ffn_hidden_size, spec.activation, spec.mlp_up.bias is not None,
                               process_group, sequence_parallel, spec.mlp_up, spec.mlp_gate, spec.mlp_down)

    @classmethod
    def from_unsharded(cls, spec: BlockSpec, process_group="tensor", sequence_parallel: bool = False):
        return cls(spec, process_group, sequence_parallel)

    def _drop(self, x):
        if self.p_drop > 0.0 and self.training:
            # the full hidden state is replicated over the tensor group: same mask on all its ranks (with
            # sequence parallelism every rank holds other tokens: private stream)
            with (get_randomizer() if self.seq_par else get_randomizer("tensor")).fork():
                return F.dropout(x, self.p_drop)
        return x

    def forward(self, x, key_padding_mask=None, position_ids=None):
        if self.post_ln:
            x = self.input_layernorm(x + self._drop(self.attention(x, key_padding_mask, position_ids)))
            return self.post_attention_layernorm(x + self._drop(self.mlp(x)))
        x = x + self._drop(self.attention(self.input_layernorm(x), key_padding_mask, position_ids))
        return x + self._drop(self.mlp(self.post_attention_layernorm(x)))


# ------------------------------------------------------------------------------------------ adapters
def _conv1d_to_linear(c) -> nn.Linear:
    """HF ``Conv1D`` stores the weight as [in, out]."""
    return _linear_from(c.weight.detach().t().contiguous(), c.bias.detach() if c.bias is not None else None)


def spec_from_gpt2_block(block, config) -> BlockSpec:
    a, m = block.attn, block.mlp
    return BlockSpec(config.hidden_size, config.num_attention_heads, m.c_fc.weight.shape[1], _conv1d_to_linear(a.c_attn),
                     _conv1d_to_linear(a.c_proj), _conv1d_to_linear(m.c_fc), _conv1d_to_linear(m.c_proj), block.ln_1,
                     block.ln_2, activation="gelu_new", causal=True, attention_dropout=config.attn_pdrop,
                     hidden_dropout=config.resid_pdrop)


def spec_from_bert_layer(layer, config) -> BlockSpec:
    sa = layer.attention.self
    w = torch.cat([sa.query.weight, sa.key.weight, sa.value.weight]).detach()
    b = torch.cat([sa.query.bias, sa.key.bias, sa.value.bias]).detach()
    return BlockSpec(config.hidden_size, config.num_attention_heads, config.intermediate_size, _linear_from(w, b),
                     layer.attention.output.dense, layer.intermediate.dense, layer.output.dense,
                     layer.attention.output.LayerNorm, layer.output.LayerNorm, activation="gelu", causal=False,
                     post_layernorm=True, attention_dropout=config.attention_probs_dropout_prob,
                     hidden_dropout=config.hidden_dropout_prob)


def spec_from_llama_layer(layer, config, rotary: Optional[Callable] = None) -> BlockSpec:
    """Hugging Face ``LlamaDecoderLayer`` (separate q/k/v and gate/up projections)."""
    a, m = layer.self_attn, layer.mlp
    w = torch.cat([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight]).detach()
    return BlockSpec(config.hidden_size, config.num_attention_heads, config.intermediate_size, _linear_from(w, None),
                     a.o_proj, m.up_proj, m.down_proj, layer.input_layernorm, layer.post_attention_layernorm,
                     mlp_gate=m.gate_proj, num_kv_heads=getattr(config, "num_key_value_heads", None),
                     activation="swiglu", causal=True, rotary=rotary)


# ------------------------------------------------------------------------ checkpointing with RNG replay
class _TPCheckpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_tensors, *args):
        ctx.fn = fn
        ctx.streams = [get_randomizer(), get_randomizer("tensor")]
        ctx.states = [(r.cpu_state.clone(), None if r.cuda_state is None else r.cuda_state.clone()) for r in ctx.streams]
        ctx.autocast = (torch.is_autocast_enabled("cuda"), torch.get_autocast_dtype("cuda")) \
            if torch.cuda.is_available() else (False, None)
        ctx.save_for_backward(*[a for a in args if isinstance(a, torch.Tensor)])
        ctx.proto = [None if isinstance(a, torch.Tensor) else a for a in args]
        with torch.no_grad():
            return fn(*args)

    @staticmethod
    def backward(ctx, *grads):
        it = iter(ctx.saved_tensors)
        args = [next(it).detach().requires_grad_(True) if p is None else p for p in ctx.proto]
        for a in args:
            if isinstance(a, torch.Tensor) and not a.is_floating_point():
                a.requires_grad_(False)
        now = [(r.cpu_state, r.cuda_state) for r in ctx.streams]
        for r, (c, g) in zip(ctx.streams, ctx.states):      # replay the dropout masks of the first pass
            r.cpu_state, r.cuda_state = c, g
        try:
            with torch.enable_grad(), torch.autocast("cuda", enabled=ctx.autocast[0], dtype=ctx.autocast[1]) \
                    if ctx.autocast[0] else torch.enable_grad():
                out = ctx.fn(*args)
        finally:
            for r, (c, g) in zip(ctx.streams, now):
                r.cpu_state, r.cuda_state = c, g
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(a.grad if isinstance(a, torch.Tensor) and a.requires_grad else None for a in args)


def tp_checkpoint(fn: Callable, *args):
    """Recompute ``fn(*args)`` in the backward pass with the tensor-parallel RNG streams restored to what they
    were in the first pass. Parameters reached through ``fn`` receive their gradients in the recomputation."""
    return _TPCheckpoint.apply(fn, len(args), *args)


__all__ = ["ParallelSelfAttention", "ParallelMLP", "ParallelTransformerLayer", "BlockSpec", "spec_from_gpt2_block",
           "spec_from_bert_layer", "spec_from_llama_layer", "tp_checkpoint"]
del math
