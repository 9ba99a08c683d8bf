"""Front end of the sm_100a flash-attention kernels (csrc/flash_attn.cu)."""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from .. import _lib


def kernels_built() -> bool:
    L = _lib.lib()
    return L is not None and L.has("atb_flash_fwd")


def supported(q, k, v, dropout_p=0.0, additive_mask=None, additive_bias=None) -> bool:
    if not _lib.use_kernels(q, k, v) or not kernels_built():
        return False
    if dropout_p != 0.0 or additive_mask is not None or additive_bias is not None:
        return False
    B, Sq, Hq, D = q.shape
    return (q.dtype == torch.bfloat16 and D == 128 and Hq % k.shape[2] == 0 and k.shape[1] % 8 == 0)


def flash_attention(q, k, v, causal=False, softmax_scale=None, glm_mask=None, pack_glm_mask=None,
                    key_padding_mask=None, cu_seqlens=None):
    raise NotImplementedError
