"""Scaled-dot-product attention with the mask family of the reference's ``FlashAttnModule``:
causal, key-padding / packed variable-length sequences, GLM break-point masks, packed GLM masks,
additive masks and biases, grouped-query heads.

Mask semantics (reference: atorch/modules/transformer/layers.py:1283-1408, docs/FA-glm.md:52-160,
atorch/npu/layers.py:9-45):

* ``causal``: row i sees columns j <= i (aligned to the bottom-right when s_q != s_k).
* ``glm_mask`` ``[B]`` int: row i sees column j iff ``j <= i`` or ``j < glm_mask[b]``.
* packed GLM mask ``[B, 2, P]`` int (row 0 starts, row 1 ends, -1 = unused): causal, plus for every
  pair (s, e) each row ``i >= s`` sees every column ``j < e``.
* ``key_padding_mask`` ``[B, S_k]``: True/1 = valid key.
* ``cu_seqlens`` (packed sequences): tokens only see keys of their own sequence.
* ``additive_mask`` / ``additive_bias``: added to the scaled scores before the softmax (a boolean
  ``additive_mask`` means True = visible). A 0 / -inf mask shared by all heads with one run of visible keys per
  row is lowered to key intervals; any other mask or bias without a gradient is added to the scores inside the
  flash kernels as one bf16 tensor (S_k a multiple of 8); a bias that needs a gradient takes the dense path.

``attention`` dispatches to the sm_100a flash-attention kernels when they are built and the
problem fits them, and evaluates the dense PyTorch reference otherwise (CPU, unusual shapes).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _lib


def build_dense_mask(B: int, Sq: int, Sk: int, device, causal: bool = False, glm_mask: Optional[torch.Tensor] = None,
                     pack_glm_mask: Optional[torch.Tensor] = None, key_padding_mask: Optional[torch.Tensor] = None,
                     cu_seqlens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Boolean ``[B, 1, Sq, Sk]`` visibility mask (True = may attend) or None if everything is visible."""
    if not causal and glm_mask is None and pack_glm_mask is None and key_padding_mask is None and cu_seqlens is None:
        return None
    i = torch.arange(Sq, device=device)[:, None] + (Sk - Sq)
    j = torch.arange(Sk, device=device)[None, :]
    if causal or glm_mask is not None or pack_glm_mask is not None:
        vis = (j <= i)[None].expand(B, Sq, Sk).clone()
    else:
        vis = torch.ones(B, Sq, Sk, dtype=torch.bool, device=device)
    if glm_mask is not None:
        vis |= j[None] < glm_mask.to(device).view(B, 1, 1)
    if pack_glm_mask is not None:
        pm = pack_glm_mask.to(device)
        for b in range(B):
            for s, e in zip(pm[b, 0].tolist(), pm[b, 1].tolist()):
                if s < 0 or e < 0:
                    continue
                vis[b, s:, :e] = True
    if key_padding_mask is not None:
        vis &= key_padding_mask.to(device).bool()[:, None, :]
    if cu_seqlens is not None:
        seg = torch.bucketize(torch.arange(Sk, device=device), cu_seqlens.to(device)[1:], right=True)
        vis &= (seg[:, None] == seg[None, :])[None]
    return vis[:, None]


def attention_reference(q, k, v, causal=False, softmax_scale=None, glm_mask=None, pack_glm_mask=None,
                        key_padding_mask=None, cu_seqlens=None, additive_mask=None, additive_bias=None,
                        dropout_p=0.0):
    """Dense fp32 attention. q: [B, Sq, Hq, D]; k, v: [B, Sk, Hkv, D]; returns [B, Sq, Hq, D]."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    qf, kf, vf = q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2)
    if Hkv != Hq:
        kf = kf.repeat_interleave(Hq // Hkv, dim=1)
        vf = vf.repeat_interleave(Hq // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if additive_bias is not None:
        s = s + additive_bias.float()
    if additive_mask is not None:
        s = s.masked_fill(~additive_mask, float("-inf")) if additive_mask.dtype == torch.bool \
            else s + additive_mask.float()
    vis = build_dense_mask(B, Sq, Sk, q.device, causal, glm_mask, pack_glm_mask, key_padding_mask, cu_seqlens)
    if vis is not None:
        s = s.masked_fill(~vis, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)  # fully masked rows produce zeros
    if dropout_p > 0.0:
        p = torch.nn.functional.dropout(p, dropout_p)
    o = torch.matmul(p, vf)
    return o.transpose(1, 2).to(q.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
              softmax_scale: Optional[float] = None, glm_mask: Optional[torch.Tensor] = None,
              pack_glm_mask: Optional[torch.Tensor] = None, key_padding_mask: Optional[torch.Tensor] = None,
              cu_seqlens: Optional[torch.Tensor] = None, additive_mask: Optional[torch.Tensor] = None,
              additive_bias: Optional[torch.Tensor] = None, dropout_p: float = 0.0) -> torch.Tensor:
    """Attention over ``[B, S, H, D]`` tensors with the mask options described in the module docstring."""
    from . import flash

    if additive_mask is not None and additive_bias is None and glm_mask is None and pack_glm_mask is None \
            and key_padding_mask is None and cu_seqlens is None and flash.supported(q, k, v, dropout_p):
        # a dense 0 / -inf (or boolean) mask that is one run of visible keys per row runs in the flash kernels
        iv = flash.intervals_from_additive_mask(additive_mask, q.shape[0], q.shape[1], k.shape[1], causal)
        if iv is not None:
            scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
            drop = flash.dropout_config(dropout_p) if dropout_p > 0.0 else None
            return flash._FlashAttn.apply(q, k, v, False, float(scale), iv[0], iv[1], drop)
    if flash.supported(q, k, v, dropout_p, additive_mask, additive_bias, key_padding_mask):
        return flash.flash_attention(q, k, v, causal=causal, softmax_scale=softmax_scale, glm_mask=glm_mask,
                                     pack_glm_mask=pack_glm_mask, key_padding_mask=key_padding_mask,
                                     cu_seqlens=cu_seqlens, dropout_p=dropout_p, additive_mask=additive_mask,
                                     additive_bias=additive_bias)
    if q.is_cuda and glm_mask is None and pack_glm_mask is None and key_padding_mask is None and cu_seqlens is None \
            and additive_mask is None and additive_bias is None and q.shape[1] == k.shape[1]:
        # library path (torch SDPA) for shapes the sm_100a kernels do not cover
        global library_calls
        library_calls += 1
        o = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p=dropout_p, is_causal=causal,
            scale=softmax_scale, enable_gqa=q.shape[2] != k.shape[2])
        return o.transpose(1, 2)
    return attention_reference(q, k, v, causal, softmax_scale, glm_mask, pack_glm_mask, key_padding_mask, cu_seqlens,
                               additive_mask, additive_bias, dropout_p)


library_calls = 0  # how often the library path above was taken (benchmarks report it)
