"""Front end of the sm_100a flash-attention kernels (csrc/flash_attn.cu, csrc/flash_attn_bwd.cu).

All masks are lowered to one per-row key interval ``[lo, hi)``:

=====================  ==========================================================
causal                 ``hi = i + 1 + (Sk - Sq)``
GLM break-point g[b]   ``hi = max(i + 1, g[b])``
packed GLM [b, 2, P]   ``hi = max(i + 1, max{e_p : s_p <= i})``
key padding            ``[lo, hi) = [first valid key, last valid key + 1)`` when the valid keys of a row are
                       contiguous (right or left padding); masks with holes are unpadded into packed
                       sequences (``cu_seqlens``) like the reference's varlen path
packed sequences       ``lo = start of the row's sequence`` (``cu_seqlens``)
=====================  ==========================================================

(Reference semantics: atorch/modules/transformer/layers.py:1283-1408, docs/FA-glm.md:52-160.)
"""
from __future__ import annotations

import collections
import ctypes
import math
from typing import Optional, Tuple

import torch

from .. import _lib


import os
import weakref

# forward kernel with two 128-row query tiles per CTA that share every K/V tile (csrc/flash_attn_v2.cu): the
# default from 256 query rows on (measured 201 us against 256 us for the single-tile kernel at S=4096, H=32,
# causal); ATB_FLASH_V2=0 keeps the single-tile kernel everywhere
FWD_TWO_TILES = os.environ.get("ATB_FLASH_V2", "1") == "1"
# backward as two kernels (dK/dV per key block + dQ per query block; no atomics, no fp32 scratch): measured 667 us
# against 696 us for the single key-block kernel at S=4096, H=32, causal. ATB_FLASH_BWD_SPLIT=0 selects the latter.
BWD_SPLIT = os.environ.get("ATB_FLASH_BWD_SPLIT", "1") == "1"
_DKV_SET = False   # ATB_FLASH_BWD_DKV=0 / 1 forces the shared-memory / transposed key-block kernel (default: by shape)


def kernels_built() -> bool:
    L = _lib.lib()
    return L is not None and L.has("atb_flash_fwd")


def backward_built() -> bool:
    L = _lib.lib()
    return L is not None and L.has("atb_flash_bwd")


def supported(q, k, v, dropout_p=0.0, additive_mask=None, additive_bias=None, key_padding_mask=None) -> bool:
    if not _lib.use_kernels(q, k, v) or not kernels_built():
        return False
    if additive_mask is not None or additive_bias is not None:
        # soft masks / biases run in the kernels when they can be read as one bf16 tensor without a gradient
        if not _lib.lib().has("atb_flash_fwd_bias") or k.shape[1] % 8 != 0:
            return False
        for t in (additive_mask, additive_bias):
            if t is not None and (t.requires_grad or t.dim() < 2 or t.dim() > 4 or t.shape[-1] != k.shape[1]
                                  or t.shape[-2] not in (1, q.shape[1])):
                return False
    if dropout_p != 0.0 and not (0.0 < dropout_p < 1.0 and _lib.lib().has("atb_flash_fwd_dropout")):
        return False
    if (q.requires_grad or k.requires_grad or v.requires_grad) and torch.is_grad_enabled() and not backward_built():
        return False
    B, Sq, Hq, D = q.shape
    ok = q.dtype == torch.bfloat16 and Hq % k.shape[2] == 0 and \
        (D == 128 or (D == 64 and _lib.lib().has("atb_flash_fwd_ex")))
    ok = ok and all(t.stride(-1) == 1 and t.stride(2) == D and t.stride(1) % 8 == 0 for t in (q, k, v))
    ok = ok and all(t.stride(0) == t.stride(1) * t.shape[1] for t in (q, k, v))
    return ok


def row_intervals(B: int, Sq: int, Sk: int, device, causal: bool = False, glm_mask=None, pack_glm_mask=None,
                  key_padding_mask=None, cu_seqlens=None) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Lower the mask arguments to int32 ``(row_lo, row_hi)`` of shape [B, Sq]; ``(None, None)`` when the
    analytic causal / full form inside the kernel is enough."""
    if glm_mask is None and pack_glm_mask is None and key_padding_mask is None and cu_seqlens is None:
        return None, None
    i = torch.arange(Sq, device=device, dtype=torch.int64)
    shift = Sk - Sq
    causal_like = causal or glm_mask is not None or pack_glm_mask is not None
    hi = (i + 1 + shift).clamp(max=Sk)[None].expand(B, Sq).clone() if causal_like else \
        torch.full((B, Sq), Sk, device=device, dtype=torch.int64)
    lo = torch.zeros(B, Sq, device=device, dtype=torch.int64)
    if glm_mask is not None:
        hi = torch.maximum(hi, glm_mask.to(device).long().view(B, 1).expand(B, Sq))
    if pack_glm_mask is not None:
        pm = pack_glm_mask.to(device).long()
        s, e = pm[:, 0], pm[:, 1]                       # [B, P]
        valid = (s >= 0) & (e >= 0)
        applies = valid[:, None, :] & (s[:, None, :] <= i[None, :, None])   # [B, Sq, P]
        ext = torch.where(applies, e[:, None, :].expand(B, Sq, -1), torch.zeros((), device=device, dtype=torch.int64))
        hi = torch.maximum(hi, ext.max(dim=-1).values)
    if cu_seqlens is not None:
        cu = cu_seqlens.to(device).long()
        seg = torch.bucketize(i, cu[1:], right=True).clamp(max=cu.numel() - 2)
        lo = torch.maximum(lo, cu[seg][None].expand(B, Sq))
        if not causal_like:
            hi = torch.minimum(hi, cu[seg + 1][None].expand(B, Sq))
    if key_padding_mask is not None:
        kp = key_padding_mask.to(device).bool()
        cnt = kp.sum(dim=1)
        first = kp.int().argmax(dim=1)
        last = Sk - 1 - kp.flip(1).int().argmax(dim=1)
        # one host sync: an interval can only describe valid keys that lie next to each other
        if not bool(((cnt == 0) | (last - first + 1 == cnt)).all()):
            raise NonContiguousKeyMask()
        last1 = torch.where(cnt > 0, last + 1, torch.zeros_like(last))
        lo = torch.maximum(lo, first.view(B, 1).expand(B, Sq))
        hi = torch.minimum(hi, last1.view(B, 1).expand(B, Sq))
    hi = hi.clamp(max=Sk)
    return lo.to(torch.int32).contiguous(), hi.to(torch.int32).contiguous()


_INTERVAL_CACHE: "collections.OrderedDict" = collections.OrderedDict()   # the layers of one forward share one mask


def intervals_from_additive_mask(additive_mask: torch.Tensor, B: int, Sq: int, Sk: int, causal: bool = False):
    """Cached front of ``_intervals_from_additive_mask``: every layer of a forward pass is given the same mask
    tensor, so the lowering (one pass over the mask and one host synchronisation) runs once per mask, not per layer."""
    key = (additive_mask.data_ptr(), tuple(additive_mask.shape), additive_mask.dtype, additive_mask._version,
           str(additive_mask.device), B, Sq, Sk, bool(causal))
    hit = _INTERVAL_CACHE.get(key)
    if hit is not None and hit[0]() is additive_mask:
        return hit[1]
    out = _intervals_from_additive_mask(additive_mask, B, Sq, Sk, causal)
    try:
        _INTERVAL_CACHE[key] = (weakref.ref(additive_mask), out)
    except TypeError:
        return out
    while len(_INTERVAL_CACHE) > 8:
        _INTERVAL_CACHE.popitem(last=False)
    return out


def _intervals_from_additive_mask(additive_mask: torch.Tensor, B: int, Sq: int, Sk: int, causal: bool = False):
    """Lower a dense mask to per-row key intervals, or return ``None`` when it is not of that form.

    ``additive_mask``: broadcastable to ``[B, 1, Sq, Sk]`` (the same for every head), either boolean (True =
    visible) or additive with entries that are 0 (visible) or <= -1e4 (hidden) — the ``-65504 * (1 - ltor_mask)``
    and ``-inf`` conventions. Causal, GLM prefix, packed-sequence and padding masks all have one contiguous run of
    visible keys per row, which is what the kernels take; a mask with soft biases or holes is left to the dense
    path. Costs one pass over the mask and one host synchronisation."""
    m = additive_mask
    if m.dim() == 4:
        if m.shape[1] != 1:
            return None
        m = m[:, 0]
    elif m.dim() == 2:
        m = m[None]
    if m.dim() != 3 or m.shape[-2:] != (Sq, Sk) or m.shape[0] not in (1, B):
        return None
    if m.dtype == torch.bool:
        vis, binary = m, None
    else:
        vis = m > -1e4
        binary = ((m == 0) | ~vis).all()
    cnt = vis.sum(-1)
    first = vis.int().argmax(-1)
    last = Sk - 1 - vis.flip(-1).int().argmax(-1)
    ok = ((cnt == 0) | (last - first + 1 == cnt)).all()
    if binary is not None:
        ok = ok & binary
    if not bool(ok):
        return None
    lo = torch.where(cnt > 0, first, torch.zeros_like(first)).expand(B, Sq)
    hi = torch.where(cnt > 0, last + 1, torch.zeros_like(last)).expand(B, Sq)
    if causal:
        i = torch.arange(Sq, device=m.device)
        hi = torch.minimum(hi, (i + 1 + (Sk - Sq)).clamp(min=0)[None])
    return lo.to(torch.int32).contiguous(), hi.to(torch.int32).contiguous()


class NonContiguousKeyMask(ValueError):
    """The valid keys of some row are not contiguous: no per-row interval describes the mask."""


def _token_stride(t: torch.Tensor) -> int:
    return t.stride(1)


def bias_config(B: int, Hq: int, Sq: int, Sk: int, additive_mask=None, additive_bias=None):
    """``(tensor, stride_b, stride_h, stride_q)`` for the bias kernels: mask and bias summed into one bf16 tensor
    of shape ``[1|B, 1|H, 1|Sq, Sk]`` (2-D = ``[Sq, Sk]``, 3-D = ``[B, Sq, Sk]``), broadcast dims with stride 0."""
    t = None
    for x in (additive_mask, additive_bias):
        if x is None:
            continue
        if x.dtype == torch.bool:
            x = torch.zeros(x.shape, dtype=torch.float32, device=x.device).masked_fill(~x, float("-inf"))
        x = x[None, None] if x.dim() == 2 else x[:, None] if x.dim() == 3 else x
        t = x.float() if t is None else t + x.float()
    t = t.to(torch.bfloat16).contiguous()
    b, h, sq, sk = t.shape
    assert b in (1, B) and h in (1, Hq) and sq in (1, Sq) and sk == Sk, (t.shape, (B, Hq, Sq, Sk))
    return t, (0 if b == 1 else h * sq * sk), (0 if h == 1 else sq * sk), (0 if sq == 1 else sk)


def dropout_config(dropout_p: float, seed=None) -> Tuple[int, int, int]:
    """``(thr16, seed_lo, seed_hi)`` for the dropout kernels: an element is dropped when its 16 hash bits are below
    ``thr16 = round(p * 65536)`` (so the effective probability is ``thr16 / 65536``). The seed pair is drawn from
    torch's CPU generator (restored by activation checkpointing, so a recomputed forward draws the same mask)
    unless given."""
    thr = min(max(int(round(dropout_p * 65536.0)), 1), 65535)
    if seed is None:
        lo, hi = torch.randint(0, 2 ** 31 - 1, (2,)).tolist()
    else:
        lo, hi = int(seed) & 0xFFFFFFFF, (int(seed) >> 32) & 0xFFFFFFFF
    return thr, lo, hi


def _hash32(x: torch.Tensor) -> torch.Tensor:
    m = 0xFFFFFFFF
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    return x ^ (x >> 16)


def dropout_keep_mask(B: int, Hq: int, Sq: int, Sk: int, drop: Tuple[int, int, int], device="cpu") -> torch.Tensor:
    """The keep mask ``[B, Hq, Sq, Sk]`` (bool) the kernels use for ``drop = (thr16, seed_lo, seed_hi)``: the
    host restatement of ``drop_row_key`` / ``drop_pair_bits`` (csrc/common.cuh), used by the tests."""
    thr, lo, hi = drop
    m = 0xFFFFFFFF
    bh = torch.arange(B * Hq, dtype=torch.int64, device=device)
    base = _hash32(lo ^ ((bh * 0x9E3779B1) & m)) ^ hi                               # [B*Hq]
    rows = torch.arange(Sq, dtype=torch.int64, device=device)
    key = _hash32((base[:, None] + ((rows * 0x85EBCA77) & m)[None]) & m)             # [B*Hq, Sq]
    pairs = torch.arange((Sk + 1) // 2, dtype=torch.int64, device=device)
    w = _hash32(key[:, :, None] ^ ((pairs * 0xC2B2AE3D) & m)[None, None])            # [B*Hq, Sq, Sk/2]
    bits = torch.stack([w & 0xFFFF, w >> 16], dim=-1).reshape(B * Hq, Sq, -1)[:, :, :Sk]
    return (bits >= thr).view(B, Hq, Sq, Sk)


def _extra_args(drop, bias, head_dim=None):
    d = drop if drop is not None else (0, 0, 0)
    extra = tuple(ctypes.c_uint(x) for x in d)
    if bias is not None:
        extra += (_lib.ptr(bias[0]),) + tuple(ctypes.c_longlong(x) for x in bias[1:])
    elif head_dim is not None:
        extra += (None, ctypes.c_longlong(0), ctypes.c_longlong(0), ctypes.c_longlong(0))
    if head_dim is not None:
        extra += (ctypes.c_int(head_dim),)
    return extra


def flash_fwd_raw(q, k, v, causal, softmax_scale, row_lo, row_hi, drop=None, bias=None):
    """Launch the forward kernel. Returns (out [B,Sq,Hq,D] bf16, lse [B,Hq,Sq] fp32). ``drop``: see
    ``dropout_config``; dropout runs in the single-tile kernel."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    out = torch.empty(B, Sq, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q.device)
    L = _lib.lib()
    # two-query-tile kernel (flash_attn_v2.cu) for long enough sequences; the single-tile kernel otherwise
    if D != 128:
        fwd, extra = L.atb_flash_fwd_ex, _extra_args(drop, bias, D)      # single-tile kernel, head dim 64
    elif bias is not None:
        fwd, extra = L.atb_flash_fwd_bias, _extra_args(drop, bias)
    elif drop is not None:
        fwd, extra = L.atb_flash_fwd_dropout, _extra_args(drop, None)
    else:
        fwd = L.atb_flash_fwd_v2 if (FWD_TWO_TILES and Sq >= 256 and L.has("atb_flash_fwd_v2")) else L.atb_flash_fwd
        extra = ()
    rc = fwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(row_lo), _lib.ptr(row_hi),
        ctypes.c_int(B), ctypes.c_int(Sq), ctypes.c_int(Sk), ctypes.c_int(Hq), ctypes.c_int(Hkv),
        ctypes.c_longlong(_token_stride(q)), ctypes.c_longlong(_token_stride(k)), ctypes.c_longlong(_token_stride(v)),
        ctypes.c_int(int(causal)), ctypes.c_float(softmax_scale), _lib.stream_ptr(),
        _lib.ptr(_lib.status_word(q.device)), *extra)
    _lib.check(rc, "atb_flash_fwd")
    return out, lse


def flash_bwd_raw(dout, q, k, v, out, lse, causal, softmax_scale, row_lo, row_hi, fused_out: bool = False,
                  drop=None, bias=None):
    """Launch the backward kernels. Returns (dq, dk, dv) shaped like q, k, v. With ``fused_out`` (and
    equal query / key-value head counts) the three are slices of ONE ``[B, S, 3*H, D]`` buffer laid out
    like a fused q|k|v projection output, so the gradient of that projection needs no concatenation."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    global _DKV_SET
    if not _DKV_SET:
        _DKV_SET = True
        if os.environ.get("ATB_FLASH_BWD_DKV", "") in ("0", "1"):
            _lib.lib().atb_flash_bwd_set_dkv(ctypes.c_int(int(os.environ["ATB_FLASH_BWD_DKV"])))
    # two kernels (dK/dV per key block, dQ per query block: no atomics, no fp32 scratch) unless
    # ATB_FLASH_BWD_SPLIT=0 asks for the single key-block kernel with TMA reduce-adds of dQ
    dq_acc = None if (BWD_SPLIT and drop is None and bias is None and D == 128) else \
        torch.zeros(B, Sq, Hq, D, dtype=torch.float32, device=q.device)
    delta = torch.empty(B, Hq, Sq, dtype=torch.float32, device=q.device)
    if fused_out and Hkv == Hq and Sq == Sk:
        fused = torch.empty(B, Sq, 3 * Hq, D, dtype=q.dtype, device=q.device)
        dq, dk, dv = fused[:, :, :Hq], fused[:, :, Hq: 2 * Hq], fused[:, :, 2 * Hq:]
    else:
        fused = None
        dq = torch.empty(B, Sq, Hq, D, dtype=q.dtype, device=q.device)
        dk = torch.empty(B, Sk, Hq, D, dtype=q.dtype, device=q.device)
        dv = torch.empty(B, Sk, Hq, D, dtype=q.dtype, device=q.device)
    dout = dout if (dout.stride(-1) == 1 and dout.stride(2) == D and dout.stride(0) == dout.stride(1) * Sq) \
        else dout.contiguous()
    if D != 128:
        bwd, extra = _lib.lib().atb_flash_bwd_ex, _extra_args(drop, bias, D)
    elif bias is not None:
        bwd, extra = _lib.lib().atb_flash_bwd_bias, _extra_args(drop, bias)
    elif drop is not None:
        bwd, extra = _lib.lib().atb_flash_bwd_dropout, _extra_args(drop, None)
    else:
        bwd, extra = _lib.lib().atb_flash_bwd, ()
    rc = bwd(
        _lib.ptr(dout), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(delta),
        _lib.ptr(dq_acc), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(row_lo), _lib.ptr(row_hi),
        ctypes.c_int(B), ctypes.c_int(Sq), ctypes.c_int(Sk), ctypes.c_int(Hq), ctypes.c_int(Hkv),
        ctypes.c_longlong(_token_stride(q)), ctypes.c_longlong(_token_stride(k)), ctypes.c_longlong(_token_stride(v)),
        ctypes.c_longlong(_token_stride(dout)), ctypes.c_longlong(_token_stride(dq)),
        ctypes.c_longlong(_token_stride(dk)), ctypes.c_int(int(causal)), ctypes.c_float(softmax_scale),
        _lib.stream_ptr(), _lib.ptr(_lib.status_word(q.device)), *extra)
    _lib.check(rc, "atb_flash_bwd")
    if Hkv != Hq:
        g = Hq // Hkv
        dk = dk.view(B, Sk, Hkv, g, D).float().sum(3).to(q.dtype)
        dv = dv.view(B, Sk, Hkv, g, D).float().sum(3).to(q.dtype)
    if fused is not None:
        return fused
    return dq, dk, dv


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, row_lo, row_hi, drop=None, bias=None):
        out, lse = flash_fwd_raw(q, k, v, causal, scale, row_lo, row_hi, drop, bias)
        ctx.save_for_backward(q, k, v, out, lse, row_lo, row_hi)
        ctx.cfg = (causal, scale, drop, bias)       # bias: (bf16 tensor, strides), not differentiated
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, row_lo, row_hi = ctx.saved_tensors
        causal, scale, drop, bias = ctx.cfg
        dq, dk, dv = flash_bwd_raw(dout, q, k, v, out, lse, causal, scale, row_lo, row_hi, drop=drop, bias=bias)
        return dq, dk, dv, None, None, None, None, None, None


def flash_attention(q, k, v, causal=False, softmax_scale=None, glm_mask=None, pack_glm_mask=None,
                    key_padding_mask=None, cu_seqlens=None, dropout_p=0.0, dropout_seed=None,
                    additive_mask=None, additive_bias=None):
    """``dropout_p``: attention dropout inside the kernels (the mask is a counter-based hash of batch, head, row
    and column, see ``dropout_keep_mask``); ``dropout_seed`` fixes the mask, otherwise torch's CPU generator
    supplies the seed."""
    B, Sq, Hq, D = q.shape
    Sk = k.shape[1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    if Sq == 1:
        causal = False   # single-query decode sees every key
    try:
        lo, hi = row_intervals(B, Sq, Sk, q.device, causal, glm_mask, pack_glm_mask, key_padding_mask, cu_seqlens)
    except NonContiguousKeyMask:
        if additive_mask is not None or additive_bias is not None:
            from .attention import attention_reference

            return attention_reference(q, k, v, causal, scale, glm_mask, pack_glm_mask, key_padding_mask, cu_seqlens,
                                       additive_mask, additive_bias, dropout_p)
        return _unpadded_attention(q, k, v, key_padding_mask, causal, scale, glm_mask, pack_glm_mask, cu_seqlens,
                                   dropout_p, dropout_seed)
    drop = dropout_config(dropout_p, dropout_seed) if dropout_p > 0.0 else None
    bias = None
    if additive_mask is not None or additive_bias is not None:
        bias = bias_config(B, Hq, Sq, Sk, additive_mask, additive_bias)
    return _FlashAttn.apply(q, k, v, bool(causal), float(scale), lo, hi, drop, bias)


def _unpadded_attention(q, k, v, key_padding_mask, causal, scale, glm_mask, pack_glm_mask, cu_seqlens,
                        dropout_p=0.0, dropout_seed=None):
    """Key-padding mask with holes (self-attention): drop the padded tokens, run the batch as packed
    sequences, put the results back (padded positions get zeros). Mirrors the reference's unpad / pad
    path (atorch/modules/transformer/layers.py:76-95,1363-1408)."""
    B, S, H, D = q.shape
    if k.shape[1] != S or glm_mask is not None or pack_glm_mask is not None or cu_seqlens is not None:
        from .attention import attention_reference

        return attention_reference(q, k, v, causal, scale, glm_mask, pack_glm_mask, key_padding_mask, cu_seqlens,
                                   dropout_p=dropout_p)
    kp = key_padding_mask.to(q.device).bool()
    idx = kp.reshape(-1).nonzero(as_tuple=False)[:, 0]
    cu = torch.zeros(B + 1, dtype=torch.int32, device=q.device)
    cu[1:] = kp.sum(1).cumsum(0)
    pick = lambda t: t.reshape(B * S, t.shape[2], D).index_select(0, idx).unsqueeze(0)
    out_p = flash_attention(pick(q), pick(k), pick(v), causal=causal, softmax_scale=scale, cu_seqlens=cu,
                            dropout_p=dropout_p, dropout_seed=dropout_seed)
    out = torch.zeros(B * S, H, D, dtype=q.dtype, device=q.device)
    out = out.index_copy(0, idx, out_p[0])
    return out.view(B, S, H, D)


class _FlashAttnQKV(torch.autograd.Function):
    """Attention on a fused projection output ``qkv [B, S, 3*H, D]`` (q heads, then k, then v). The
    backward emits one fused gradient tensor in the same layout: no slice-backward zero fills or adds."""

    @staticmethod
    def forward(ctx, qkv, H, causal, scale, row_lo, row_hi, cached):
        q, k, v = qkv[:, :, :H], qkv[:, :, H: 2 * H], qkv[:, :, 2 * H:]
        if cached is not None:
            out, lse = cached          # output and log-sum-exp kept from the first pass of a checkpointed block
        else:
            out, lse = flash_fwd_raw(q, k, v, causal, scale, row_lo, row_hi)
        ctx.save_for_backward(qkv, out, lse, row_lo, row_hi)
        ctx.cfg = (H, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, row_lo, row_hi = ctx.saved_tensors
        H, causal, scale = ctx.cfg
        q, k, v = qkv[:, :, :H], qkv[:, :, H: 2 * H], qkv[:, :, 2 * H:]
        dqkv = flash_bwd_raw(dout, q, k, v, out, lse, causal, scale, row_lo, row_hi, fused_out=True)
        return dqkv, None, None, None, None, None, None


def flash_attention_qkv(qkv: torch.Tensor, num_heads: int, causal: bool = True, softmax_scale=None,
                        recompute_cache=None, **mask_kwargs):
    """qkv: ``[B, S, 3*num_heads, D]``; returns ``[B, S, num_heads, D]``.

    ``recompute_cache`` (an ``OrderedDict`` owned by the calling layer) lets an activation-checkpointed
    block keep the attention output and log-sum-exp of its first (no-grad) pass: that pass stores
    ``(out, lse)`` under the pass token of its checkpoint node (utils/checkpoint.py), the recomputation
    of the same node takes the entry with the same token and skips the forward kernel. A forward that
    is not the first pass of a checkpointed block has no token and neither stores nor reads, and an
    entry whose backward never ran is evicted once more than ``RECOMPUTE_CACHE_LIMIT`` are held.
    32 MB per layer at 7B scale buys one attention forward per layer per step."""
    from ..utils.checkpoint import current_pass

    B, S, _, D = qkv.shape
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    try:
        lo, hi = row_intervals(B, S, S, qkv.device, causal, mask_kwargs.get("glm_mask"),
                               mask_kwargs.get("pack_glm_mask"), mask_kwargs.get("key_padding_mask"),
                               mask_kwargs.get("cu_seqlens"))
    except NonContiguousKeyMask:
        H = num_heads
        return flash_attention(qkv[:, :, :H], qkv[:, :, H: 2 * H], qkv[:, :, 2 * H:], causal=causal,
                               softmax_scale=softmax_scale, **mask_kwargs)
    cached = None
    cur = current_pass() if recompute_cache is not None else None
    if cur is not None:
        token, is_recompute = cur
        if not is_recompute and not torch.is_grad_enabled():
            H = num_heads
            out, lse = flash_fwd_raw(qkv[:, :, :H], qkv[:, :, H: 2 * H], qkv[:, :, 2 * H:], bool(causal), float(scale),
                                     lo, hi)
            recompute_cache[token] = (out, lse)
            while len(recompute_cache) > RECOMPUTE_CACHE_LIMIT:
                recompute_cache.popitem(last=False)
            return out
        if is_recompute:
            cached = recompute_cache.pop(token, None)
            if cached is not None and cached[0].shape != (B, S, num_heads, D):
                cached = None
    return _FlashAttnQKV.apply(qkv, num_heads, bool(causal), float(scale), lo, hi, cached)


RECOMPUTE_CACHE_LIMIT = 16   # first passes in flight per layer (pipeline micro-batches) before eviction
