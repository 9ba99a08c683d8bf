"""Llama-family decoder (Llama-2 7B/13B, 1.3B, GQA variants) on the atorch_b200 operators.

The block keeps fused parameters (``qkv_proj`` = q|k|v rows, ``gate_up_proj`` = gate|up rows) so
that each is one tcgen05 GEMM; :func:`to_hf_state_dict` / :func:`from_hf_state_dict` convert to and
from the Hugging Face parameter names (``q_proj``, ``k_proj``, ``v_proj``, ``gate_proj``,
``up_proj``), so checkpoints interchange with the models the reference trains
(examples/llama2/train_llama2_dummy_data.py builds ``transformers.LlamaForCausalLM``).

Per-layer dataflow (all bf16, fp32 accumulation inside the kernels):
    x   = rms_norm(h)                      csrc/norm.cu
    qkv = x @ Wqkv^T                       csrc/gemm_bf16.cu
    qkv = rope(qkv) on the q and k heads   csrc/elementwise.cu
    a   = attention(q, k, v, causal)       csrc/flash_attn.cu
    h   = h + a @ Wo^T                     GEMM epilogue accumulates into the residual stream
    x   = rms_norm(h)
    act = swiglu(x @ Wgu^T)
    h   = h + act @ Wdown^T
"""
from __future__ import annotations

import collections
import math
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import flash
from ..utils.checkpoint import checkpoint_module


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False
    gradient_checkpointing: bool = False
    reuse_attention_in_recompute: bool = True   # checkpointed blocks keep attention out/lse instead of recomputing

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @staticmethod
    def llama2_7b(**kw) -> "LlamaConfig":
        return LlamaConfig(32000, 4096, 11008, 32, 32, 32, 4096, **kw)

    @staticmethod
    def llama2_13b(**kw) -> "LlamaConfig":
        return LlamaConfig(32000, 5120, 13824, 40, 40, 40, 4096, **kw)

    @staticmethod
    def llama_1p3b(**kw) -> "LlamaConfig":
        return LlamaConfig(32000, 2048, 5504, 24, 16, 16, 2048, **kw)

    @staticmethod
    def tiny(**kw) -> "LlamaConfig":
        d = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                 num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256)
        d.update(kw)
        return LlamaConfig(**d)

    def num_parameters(self) -> int:
        h, f, v, L = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        kv = self.num_key_value_heads * self.head_dim
        per_layer = h * (h + 2 * kv) + h * h + 3 * h * f + 2 * h
        return L * per_layer + v * h * (1 if self.tie_word_embeddings else 2) + h

    def flops_per_token(self, seq_len: int, recompute: bool = False, attention_recompute: bool = True) -> float:
        """Megatron-convention matmul FLOPs per token of one training step (fwd + bwd = 3x fwd; the
        layer part counts 4x with activation recomputation), as in
        examples/llama2/example_utils.py:146-183 of the reference. With ``attention_recompute=False``
        the attention product is counted 3x even under recomputation: blocks that keep the attention
        output and log-sum-exp of their first pass do not execute it a second time."""
        h, f, v, L = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        kv = self.num_key_value_heads * self.head_dim
        proj = 2 * h * (h + 2 * kv) + 2 * h * h + 6 * h * f
        attn = 4 * seq_len * h
        head = 2 * h * v
        mult = 4 if recompute else 3
        return L * (proj * mult + attn * (mult if attention_recompute else 3)) + head * 3


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def reset_parameters(self):
        nn.init.ones_(self.weight)

    def forward(self, x, residual=None, carry=False):
        return ops.rms_norm(x, self.weight, self.eps, residual, carry)


class LlamaDecoderLayer(nn.Module):
    # parameters whose gradients are only ever written by this package's kernels (GEMM epilogue, norm
    # column sums): sharded engines may skip zero-filling their gradient buffers (looked up by name
    # after materialisation, since moving a module off the meta device re-creates its Parameters)
    _atb_direct_grad_params = ("qkv_proj.weight", "o_proj.weight", "gate_up_proj.weight", "down_proj.weight",
                               "input_layernorm.weight", "post_attention_layernorm.weight")

    def __init__(self, config: LlamaConfig, layer_idx: int = 0):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        h, d = config.hidden_size, config.head_dim
        self.n_q, self.n_kv = config.num_attention_heads, config.num_key_value_heads
        self.input_layernorm = RMSNorm(h, config.rms_norm_eps)
        self.qkv_proj = nn.Linear(h, (self.n_q + 2 * self.n_kv) * d, bias=False)
        self.o_proj = nn.Linear(self.n_q * d, h, bias=False)
        self.post_attention_layernorm = RMSNorm(h, config.rms_norm_eps)
        self.gate_up_proj = nn.Linear(h, 2 * config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, h, bias=False)
        self._attn_cache = collections.OrderedDict()   # pass token -> (out, lse), see ops/flash.py

    @staticmethod
    def _proj(mod: nn.Module, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Plain linears go straight to the fused GEMM (+ residual epilogue); replaced modules
        (tensor-parallel, fp8) keep their own forward."""
        if type(mod) is nn.Linear:
            return ops.linear(x, mod.weight, mod.bias, residual)
        y = mod(x)
        return y if residual is None else residual + y

    def forward(self, h: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                positions: Optional[torch.Tensor] = None, attn_kwargs: Optional[dict] = None) -> torch.Tensor:
        B, S, _ = h.shape
        d = self.config.head_dim
        # carry=True: h comes back as a second output, so that its two gradients (norm path, residual path)
        # are added inside the norm's backward kernel
        pre = type(self.input_layernorm) is RMSNorm and type(self.post_attention_layernorm) is RMSNorm
        x, h = self.input_layernorm(h, carry=True) if pre else (self.input_layernorm(h), h)
        qkv = self._proj(self.qkv_proj, x)
        S = qkv.shape[1]      # the projection may have gathered a sequence-sharded input (sequence parallelism)
        qkv = ops.rope(qkv, cos, sin, self.n_q + self.n_kv, d, positions, inplace=True)   # qkv is read by nothing else
        qkv = qkv.view(B, S, self.n_q + 2 * self.n_kv, d)
        q = qkv[:, :, : self.n_q]
        k = qkv[:, :, self.n_q: self.n_q + self.n_kv]
        v = qkv[:, :, self.n_q + self.n_kv:]
        kw = attn_kwargs or {"causal": True}
        if self.n_q == self.n_kv and flash.supported(q, k, v, kw.get("dropout_p", 0.0), kw.get("additive_mask"),
                                                     kw.get("additive_bias")) and flash.backward_built():
            cache = self._attn_cache if (self.training and self.config.reuse_attention_in_recompute) else None
            a = flash.flash_attention_qkv(qkv, self.n_q, recompute_cache=cache, **kw)   # fused gradient out
        else:
            a = ops.attention(q, k, v, **kw)
        h = self._proj(self.o_proj, a.reshape(B, S, self.n_q * d), h)
        x, h = self.post_attention_layernorm(h, carry=True) if pre else (self.post_attention_layernorm(h), h)
        if type(self.gate_up_proj) is nn.Linear and self.gate_up_proj.bias is None:
            act = ops.linear_swiglu(x, self.gate_up_proj.weight)      # SwiGLU in the GEMM epilogue
        else:
            act = ops.swiglu(self._proj(self.gate_up_proj, x))
        h = self._proj(self.down_proj, act, h)
        return h


class LlamaModel(nn.Module):
    """Causal LM: ``forward(input_ids, labels=None)`` returns ``(loss, logits)`` like the HF model the
    reference benchmarks (labels are shifted inside, mean over non-ignored tokens)."""

    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([LlamaDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.embed_tokens.weight
        self._atb_direct_grad_params = ("norm.weight",) if config.tie_word_embeddings else \
            ("norm.weight", "lm_head.weight")
        self._rope_cache: Dict = {}
        self.apply(self._init_weights)

    def _init_weights(self, m):
        std = self.config.initializer_range
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=std)

    def rope(self, seq_len: int, device) -> tuple:
        key = (seq_len, str(device))
        if key not in self._rope_cache:
            self._rope_cache = {key: ops.rope_tables(seq_len, self.config.head_dim, self.config.rope_theta, device)}
        return self._rope_cache[key]

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                positions: Optional[torch.Tensor] = None, attn_kwargs: Optional[dict] = None,
                return_logits: bool = True):
        B, S = input_ids.shape
        cos, sin = self.rope(S, input_ids.device)
        h = self.embed_tokens(input_ids)
        for layer in self.layers:
            if self.config.gradient_checkpointing and self.training and torch.is_grad_enabled():
                h = checkpoint_module(layer, h, cos, sin, positions, attn_kwargs)
            else:
                h = layer(h, cos, sin, positions, attn_kwargs)
        h = self.norm(h)
        logits = ops.linear(h, self.lm_head.weight)
        loss = None
        if labels is not None:
            loss = causal_lm_loss(logits, labels)
        return (loss, logits if return_logits else None)


def causal_lm_loss(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Next-token loss: logits[:, :-1] against labels[:, 1:], mean over non-ignored positions."""
    B, S, V = logits.shape
    shifted = torch.full_like(labels, ignore_index)
    shifted[:, :-1] = labels[:, 1:]
    per_tok = ops.cross_entropy(logits.view(B * S, V), shifted.reshape(B * S), ignore_index=ignore_index,
                                inplace_backward=True)
    n = (shifted != ignore_index).sum().clamp(min=1)
    return per_tok.sum() / n


_FUSED = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj")}


def to_hf_state_dict(model: LlamaModel) -> Dict[str, torch.Tensor]:
    """State dict under Hugging Face ``LlamaForCausalLM`` names."""
    cfg = model.config
    d = cfg.head_dim
    out = {}
    for name, t in model.state_dict().items():
        if name.startswith("layers."):
            _, idx, rest = name.split(".", 2)
            pre = f"model.layers.{idx}."
            if rest == "qkv_proj.weight":
                nq, nkv = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
                out[pre + "self_attn.q_proj.weight"] = t[:nq]
                out[pre + "self_attn.k_proj.weight"] = t[nq: nq + nkv]
                out[pre + "self_attn.v_proj.weight"] = t[nq + nkv:]
            elif rest == "gate_up_proj.weight":
                f = cfg.intermediate_size
                out[pre + "mlp.gate_proj.weight"] = t[:f]
                out[pre + "mlp.up_proj.weight"] = t[f:]
            elif rest == "o_proj.weight":
                out[pre + "self_attn.o_proj.weight"] = t
            elif rest == "down_proj.weight":
                out[pre + "mlp.down_proj.weight"] = t
            else:
                out[pre + rest] = t
        elif name == "lm_head.weight":
            out[name] = t
        else:
            out["model." + name] = t
    return out


def from_hf_state_dict(model: LlamaModel, sd: Dict[str, torch.Tensor]) -> None:
    """Load a Hugging Face ``LlamaForCausalLM`` state dict into the fused layout."""
    own = {}
    L = model.config.num_hidden_layers
    for i in range(L):
        pre = f"model.layers.{i}."
        own[f"layers.{i}.qkv_proj.weight"] = torch.cat(
            [sd[pre + f"self_attn.{n}.weight"] for n in _FUSED["qkv_proj"]], dim=0)
        own[f"layers.{i}.gate_up_proj.weight"] = torch.cat(
            [sd[pre + f"mlp.{n}.weight"] for n in _FUSED["gate_up_proj"]], dim=0)
        own[f"layers.{i}.o_proj.weight"] = sd[pre + "self_attn.o_proj.weight"]
        own[f"layers.{i}.down_proj.weight"] = sd[pre + "mlp.down_proj.weight"]
        own[f"layers.{i}.input_layernorm.weight"] = sd[pre + "input_layernorm.weight"]
        own[f"layers.{i}.post_attention_layernorm.weight"] = sd[pre + "post_attention_layernorm.weight"]
    own["embed_tokens.weight"] = sd["model.embed_tokens.weight"]
    own["norm.weight"] = sd["model.norm.weight"]
    own["lm_head.weight"] = sd.get("lm_head.weight", sd["model.embed_tokens.weight"])
    model.load_state_dict(own)
