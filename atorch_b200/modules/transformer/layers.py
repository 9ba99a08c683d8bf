"""Attention modules: ``FlashAttnModule`` (the unified attention API) and drop-in replacements for
Hugging Face / torch attention blocks that route their core through it.

``FlashAttnModule.forward(q, k, v, key_padding_mask, glm_mask, additive_mask, additive_bias)`` takes
``[batch, seq, heads, head_dim]`` tensors. Mask arguments:

* ``key_padding_mask`` ``[B, S]``: bool / 0-1 = valid-key mask; integer values > 1 mean "lengths of the
  sequences concatenated in this row" (``[[3, 2, 0, 0, 0]]`` = a 3-token and a 2-token sequence), in
  which case tokens only attend inside their own sequence;
* ``glm_mask`` ``[B]`` break points or ``[B, 2, P]`` packed (start, end) pairs; requires ``causal``;
* ``additive_mask`` ``[B, H|1, Sq|1, Sk]`` / ``additive_bias`` ``[1, H, Sq, Sk]``: added to the scores
  (not combined with causal / padding masks);
* a single query (``Sq == 1``, decoding) always sees every key.

(Reference: atorch/modules/transformer/layers.py:1283-1408 for the API, :806-1170,1411-1706 for the
Hugging Face variants.)
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn

from ... import ops


def lengths_to_intervals(mask_in_length: torch.Tensor, causal: bool):
    """``[B, S]`` length-encoded rows -> int32 (row_lo, row_hi): row i of a sequence [s, e) sees
    [s, i+1) when causal else [s, e); padding rows see nothing."""
    B, S = mask_in_length.shape
    lens = mask_in_length.long()
    ends = lens.cumsum(1)                                   # [B, S] running end of each listed sequence
    starts = ends - lens
    pos = torch.arange(S, device=lens.device)[None, :, None]            # [1, S, 1]
    inside = (pos >= starts[:, None, :]) & (pos < ends[:, None, :]) & (lens[:, None, :] > 0)   # [B, S, n]
    any_in = inside.any(-1)
    idx = inside.float().argmax(-1)
    lo = torch.gather(starts, 1, idx)
    hi_seq = torch.gather(ends, 1, idx)
    hi = torch.minimum(hi_seq, torch.arange(1, S + 1, device=lens.device)[None]) if causal else hi_seq
    lo = torch.where(any_in, lo, torch.zeros_like(lo))
    hi = torch.where(any_in, hi, torch.zeros_like(hi))
    return lo.to(torch.int32).contiguous(), hi.to(torch.int32).contiguous()


class FlashAttnModule(nn.Module):
    def __init__(self, causal: bool = False, softmax_scale: Optional[float] = None, attention_dropout: float = 0.0,
                 use_fa3: bool = False):
        super().__init__()
        self.causal, self.softmax_scale, self.attention_dropout = causal, softmax_scale, attention_dropout
        self.use_fa3 = use_fa3     # accepted for compatibility; there is one kernel family here

    def forward(self, q, k, v, key_padding_mask=None, glm_mask=None, additive_mask=None, additive_bias=None):
        b, s_q, nh, hs = q.shape
        s_k = k.shape[1]
        dropout_p = self.attention_dropout if self.training else 0.0
        if s_q == 1:
            causal = False
        else:
            assert s_q == s_k or not self.causal, \
                f"only single-query decoding may have uneven lengths, got q {s_q} / k {s_k}"
            causal = self.causal
        kw: Dict = dict(causal=causal, softmax_scale=self.softmax_scale, dropout_p=dropout_p)
        if glm_mask is not None:
            assert self.causal, "causal must be True for glm_mask"
            if glm_mask.dim() == 1:
                kw["glm_mask"] = glm_mask
            else:
                kw["pack_glm_mask"] = glm_mask
        if additive_mask is not None or additive_bias is not None:
            assert not self.causal and key_padding_mask is None, "no causal/padding mask next to an additive mask"
            kw.update(additive_mask=additive_mask, additive_bias=additive_bias)
        if key_padding_mask is not None and not bool(key_padding_mask.bool().all()):
            if key_padding_mask.dtype != torch.bool and bool((key_padding_mask > 1).any()):
                return self._concatenated(q, k, v, key_padding_mask, kw)
            if s_q == 1:
                kw["key_padding_mask"] = key_padding_mask
            else:
                kw["key_padding_mask"] = key_padding_mask
        return ops.attention(q, k, v, **kw)

    def _concatenated(self, q, k, v, mask_in_length, kw):
        from ...ops import flash

        lo, hi = lengths_to_intervals(mask_in_length, kw["causal"])
        if flash.supported(q, k, v, kw["dropout_p"]):
            scale = kw["softmax_scale"] or 1.0 / math.sqrt(q.shape[-1])
            drop = flash.dropout_config(kw["dropout_p"]) if kw["dropout_p"] > 0.0 else None
            return flash._FlashAttn.apply(q, k, v, False, float(scale), lo, hi, drop)
        B, S = mask_in_length.shape
        j = torch.arange(S, device=q.device)
        vis = (j[None, None, :] >= lo[:, :, None]) & (j[None, None, :] < hi[:, :, None])
        add = torch.zeros(B, 1, S, S, device=q.device, dtype=torch.float32).masked_fill(~vis[:, None], float("-inf"))
        return ops.attention_reference(q, k, v, False, kw["softmax_scale"], additive_mask=add,
                                       dropout_p=kw["dropout_p"])


def _causal_attention(core: "FlashAttnModule", q, k, v, attention_mask):
    """Causal self-attention as the Hugging Face decoder layers call it: ``attention_mask`` is None, a ``[B, S]``
    key-padding mask, or the ``[B, 1, S, S]`` causal-plus-padding mask (additive or boolean) that the model builds
    once per forward; the 4-D form already contains the causal structure and is lowered to key intervals once per
    mask tensor (ops.flash.intervals_from_additive_mask)."""
    if attention_mask is not None and attention_mask.dim() == 4:
        p = core.attention_dropout if core.training else 0.0
        return ops.attention(q, k, v, causal=False, softmax_scale=core.softmax_scale, additive_mask=attention_mask,
                             dropout_p=p)
    kp = attention_mask if (attention_mask is not None and attention_mask.dim() == 2) else None
    return core(q, k, v, key_padding_mask=kp)


def hf_classes() -> dict:
    """Hugging Face attention classes that can be replaced, if transformers is importable."""
    out = {}
    try:
        from transformers.models.llama.modeling_llama import LlamaAttention
        out["LlamaAttention"] = LlamaAttention
    except Exception:
        pass
    try:
        from transformers.models.bert.modeling_bert import BertAttention
        out["BertAttention"] = BertAttention
    except Exception:
        pass
    try:
        from transformers.models.gpt2.modeling_gpt2 import GPT2Attention
        out["GPT2Attention"] = GPT2Attention
    except Exception:
        pass
    try:
        from transformers.models.clip.modeling_clip import CLIPAttention
        out["CLIPAttention"] = CLIPAttention
    except Exception:
        pass
    return out


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class LlamaAttentionFA(nn.Module):
    """Replacement for ``transformers`` ``LlamaAttention`` keeping its parameters (q/k/v/o_proj) and
    call signature ``(hidden_states, position_embeddings, attention_mask, ...) -> (out, None)``."""

    def __init__(self, src: nn.Module, **kwargs):
        super().__init__()
        self.config = src.config
        self.layer_idx = getattr(src, "layer_idx", None)
        self.head_dim = getattr(src, "head_dim", src.config.hidden_size // src.config.num_attention_heads)
        self.num_heads = src.config.num_attention_heads
        self.num_key_value_heads = getattr(src.config, "num_key_value_heads", self.num_heads)
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = src.q_proj, src.k_proj, src.v_proj, src.o_proj
        self.attn = FlashAttnModule(causal=True, attention_dropout=getattr(src, "attention_dropout", 0.0))

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None,
                cache_position=None, **kwargs):
        B, S, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(B, S, self.num_heads, self.head_dim)
        k = self.k_proj(hidden_states).view(B, S, self.num_key_value_heads, self.head_dim)
        v = self.v_proj(hidden_states).view(B, S, self.num_key_value_heads, self.head_dim)
        if position_embeddings is not None:
            cos, sin = position_embeddings
            cos, sin = cos.unsqueeze(2), sin.unsqueeze(2)
            q = q * cos + _rotate_half(q) * sin
            k = k * cos + _rotate_half(k) * sin
        out = _causal_attention(self.attn, q.contiguous(), k.contiguous(), v.contiguous(), attention_mask)
        return self.o_proj(out.reshape(B, S, -1)), None


class MultiheadAttentionFA(nn.MultiheadAttention):
    """``nn.MultiheadAttention`` (self-attention, batch_first or not) on ``FlashAttnModule``."""

    @classmethod
    def from_module(cls, src: nn.MultiheadAttention, **kwargs):
        m = cls(src.embed_dim, src.num_heads, dropout=src.dropout, bias=src.in_proj_bias is not None,
                batch_first=src.batch_first, device=src.in_proj_weight.device, dtype=src.in_proj_weight.dtype)
        m.load_state_dict(src.state_dict())
        return m

    def forward(self, query, key, value, key_padding_mask=None, need_weights=False, attn_mask=None,
                average_attn_weights=True, is_causal=False):
        if need_weights or attn_mask is not None or self.in_proj_weight is None or query is not key or key is not value:
            return super().forward(query, key, value, key_padding_mask=key_padding_mask, need_weights=need_weights,
                                   attn_mask=attn_mask, average_attn_weights=average_attn_weights, is_causal=is_causal)
        x = query if self.batch_first else query.transpose(0, 1)
        B, S, E = x.shape
        qkv = nn.functional.linear(x, self.in_proj_weight, self.in_proj_bias).view(B, S, 3, self.num_heads, -1)
        core = FlashAttnModule(causal=is_causal, attention_dropout=self.dropout)
        core.train(self.training)
        kp = None if key_padding_mask is None else ~key_padding_mask.bool()     # torch: True = ignore
        out = core(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], key_padding_mask=kp)
        out = self.out_proj(out.reshape(B, S, E))
        return (out if self.batch_first else out.transpose(0, 1)), None


class BertAttentionFA(nn.Module):
    """Replacement for ``transformers`` ``BertAttention`` (self-attention + output block)."""

    def __init__(self, src: nn.Module, **kwargs):
        super().__init__()
        self.self = src.self
        self.output = src.output
        self.num_heads = src.self.num_attention_heads
        self.head_dim = src.self.attention_head_size
        self.attn = FlashAttnModule(causal=False, attention_dropout=getattr(src.self.dropout, "p", 0.0))

    def forward(self, hidden_states, attention_mask=None, *args, **kwargs):
        B, S, _ = hidden_states.shape
        s = self.self
        q = s.query(hidden_states).view(B, S, self.num_heads, self.head_dim)
        k = s.key(hidden_states).view(B, S, self.num_heads, self.head_dim)
        v = s.value(hidden_states).view(B, S, self.num_heads, self.head_dim)
        kp = None
        if attention_mask is not None:
            # HF passes [B, 1, 1, S] (or [B, 1, S, S] whose rows agree for a padding mask): additive (0 = keep, large
            # negative = drop) or boolean (True = keep)
            m = attention_mask[:, 0, -1] if attention_mask.dim() == 4 else attention_mask.reshape(B, -1)[:, -S:]
            kp = m if m.dtype == torch.bool else (m >= 0)
        ctx = self.attn(q, k, v, key_padding_mask=kp).reshape(B, S, -1)
        # (output, attention weights): recent transformers versions unpack two values
        return self.output(ctx, hidden_states), None


class GPT2AttentionFA(nn.Module):
    """Replacement for ``transformers`` ``GPT2Attention`` (fused ``c_attn`` / ``c_proj`` Conv1D weights)."""

    def __init__(self, src: nn.Module, **kwargs):
        super().__init__()
        self.c_attn, self.c_proj = src.c_attn, src.c_proj
        self.num_heads, self.head_dim = src.num_heads, src.head_dim
        self.resid_dropout = src.resid_dropout
        self.attn = FlashAttnModule(causal=True, attention_dropout=getattr(src.attn_dropout, "p", 0.0))

    def forward(self, hidden_states, *args, attention_mask=None, **kwargs):
        B, S, E = hidden_states.shape
        q, k, v = self.c_attn(hidden_states).split(E, dim=2)
        shp = (B, S, self.num_heads, self.head_dim)
        if attention_mask is None and len(args) >= 2 and torch.is_tensor(args[1]):
            attention_mask = args[1]          # (hidden_states, past_key_values, attention_mask, ...) given by position
        out = _causal_attention(self.attn, q.reshape(shp), k.reshape(shp), v.reshape(shp), attention_mask)
        return self.resid_dropout(self.c_proj(out.reshape(B, S, E))), None


class CLIPAttentionFA(nn.Module):
    """Replacement for ``transformers`` ``CLIPAttention``."""

    def __init__(self, src: nn.Module, **kwargs):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = src.q_proj, src.k_proj, src.v_proj, src.out_proj
        self.num_heads, self.head_dim = src.num_heads, src.head_dim
        self.attn = FlashAttnModule(causal=False, attention_dropout=getattr(src, "dropout", 0.0))

    def forward(self, hidden_states, attention_mask=None, causal_attention_mask=None, **kwargs):
        # the text tower passes its causal (and padding) mask as a [B, 1, S, S] tensor, additive or boolean, in
        # ``attention_mask`` (older transformers: a second ``causal_attention_mask``); the vision tower passes none.
        # A mask with one run of visible keys per row becomes key intervals inside ops.attention.
        B, S, E = hidden_states.shape
        shp = (B, S, self.num_heads, self.head_dim)
        mask = None
        for m in (attention_mask, causal_attention_mask):
            if m is None:
                continue
            if mask is None:
                mask = m
            else:
                to_add = lambda t: torch.zeros(t.shape, device=t.device).masked_fill(~t, float("-inf")) \
                    if t.dtype == torch.bool else t.float()
                mask = to_add(mask) + to_add(m)
        core = self.attn
        core.causal = False
        out = core(self.q_proj(hidden_states).view(shp), self.k_proj(hidden_states).view(shp),
                   self.v_proj(hidden_states).view(shp), additive_mask=mask).reshape(B, S, E)
        return self.out_proj(out), None


class HFGLMSelfAttentionFA(nn.Module):
    """Self-attention of the Hugging Face GLM models (``modeling_glm.py`` of THUDM/glm-10b: fused
    ``query_key_value`` projection, ``dense`` output projection, attention and output dropout) with the flash
    kernels. Built from a config or from an existing GLM ``SelfAttention`` module, whose parameters it keeps.

    ``forward(hidden_states [b, s, h], ltor_mask [b, 1, s, s] (1 = visible), mem=None)``: the left-to-right mask
    of GLM (bidirectional prefix, causal tail, per-sample separators) has one run of visible keys per row, so it is
    lowered to key intervals (``ops.flash.intervals_from_additive_mask``) instead of being added to the scores;
    any other mask takes the dense path. (Reference: atorch/modules/transformer/layers.py:1513-1632.)"""

    def __init__(self, config=None, src_module: Optional[nn.Module] = None):
        super().__init__()
        if src_module is not None:
            self.hidden_size = src_module.hidden_size
            self.num_attention_heads = src_module.num_attention_heads
            self.attention_scale = getattr(src_module, "attention_scale", 1.0)
            self.query_key_value, self.dense = src_module.query_key_value, src_module.dense
            self.attention_dropout = nn.Dropout(src_module.attention_dropout.p)
            self.output_dropout = nn.Dropout(src_module.output_dropout.p)
        else:
            self.hidden_size = getattr(config, "hidden_size", 4096)
            self.num_attention_heads = getattr(config, "num_attention_heads", 64)
            self.attention_scale = getattr(config, "attention_scale", 1.0)
            self.query_key_value = nn.Linear(self.hidden_size, 3 * self.hidden_size)
            self.dense = nn.Linear(self.hidden_size, self.hidden_size)
            self.attention_dropout = nn.Dropout(getattr(config, "attention_dropout_prob", 0.1))
            self.output_dropout = nn.Dropout(getattr(config, "output_dropout_prob", 0.1))
        assert self.hidden_size % self.num_attention_heads == 0
        self.hidden_size_per_attention_head = self.hidden_size // self.num_attention_heads

    @classmethod
    def from_module(cls, src: nn.Module, **kwargs):
        return cls(src_module=src)

    def forward(self, hidden_states, ltor_mask, mem=None):
        B, S, _ = hidden_states.shape
        x = hidden_states if mem is None else torch.cat((mem, hidden_states), 1)
        q, k, v = self.query_key_value(x).chunk(3, dim=-1)
        if mem is not None:
            q = q[:, -S:]
        heads = lambda t: t.reshape(B, t.shape[1], self.num_attention_heads, self.hidden_size_per_attention_head)
        p = self.attention_dropout.p if self.training else 0.0
        ctx = ops.attention(heads(q), heads(k), heads(v), additive_mask=ltor_mask > 0.5 if ltor_mask.dtype != torch.bool
                            else ltor_mask, dropout_p=p)
        return self.output_dropout(self.dense(ctx.reshape(B, S, self.hidden_size)))
