"""RoPE, SwiGLU and bias-gather-add on the sm_100a elementwise kernels.

Reference counterparts: atorch/kernels/triton_jit/rope.py:4-10, swiglu.py:4-11 (liger Triton
kernels) and atorch/kernels/triton_jit/bias_gather_add.py:13-160.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import _lib


def rope_tables(seq_len: int, head_dim: int, base: float = 10000.0, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables ``[seq_len, head_dim // 2]`` (HF Llama rotate-half convention)."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32, device=device)
    f = torch.outer(t, inv)
    return f.cos().contiguous(), f.sin().contiguous()


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, nheads: int, head_dim: int,
                   positions: Optional[torch.Tensor] = None, backward: bool = False) -> torch.Tensor:
    """x: [..., S, W] where the first ``nheads*head_dim`` columns are rotated. Returns a new tensor."""
    T = x.shape[:-1].numel()
    S = cos.shape[0]
    x2 = x.reshape(T, x.shape[-1]).clone()
    pos = positions.reshape(T).long() if positions is not None else (torch.arange(T, device=x.device) % S)
    c = cos[pos].unsqueeze(1).float()
    s = sin[pos].unsqueeze(1).float() * (-1.0 if backward else 1.0)
    h = x2[:, : nheads * head_dim].reshape(T, nheads, head_dim).float()
    x1, xx2 = h[..., : head_dim // 2], h[..., head_dim // 2:]
    o = torch.cat([x1 * c - xx2 * s, xx2 * c + x1 * s], dim=-1)
    x2[:, : nheads * head_dim] = o.reshape(T, nheads * head_dim).to(x.dtype)
    return x2.view(x.shape)


def _rope_launch(dst2, src2, cos, sin, positions, nheads, head_dim, backward):
    """dst2 = rope(src2) (rows = tokens); the columns after the rotated heads are copied through."""
    T, W = dst2.shape
    rc = _lib.lib().atb_rope(_lib.ptr(dst2), _lib.ptr(src2), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(positions),
                             ctypes.c_longlong(T), ctypes.c_int(cos.shape[0]), ctypes.c_int(nheads),
                             ctypes.c_int(head_dim), ctypes.c_longlong(dst2.stride(0)),
                             ctypes.c_longlong(src2.stride(0)), ctypes.c_int(W - nheads * head_dim),
                             ctypes.c_int(int(backward)), _lib.stream_ptr())
    _lib.check(rc, "atb_rope")


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, positions, nheads, head_dim, inplace):
        ctx.save_for_backward(cos, sin, positions)
        ctx.cfg = (nheads, head_dim, inplace)
        if inplace and x.stride(-1) == 1 and x.is_contiguous():
            # rotate the q / k heads where they are: the untouched columns (v heads) cost no traffic. The result
            # is a second tensor over x's storage rather than x marked dirty: x is usually a view made inside the
            # projection's autograd function, which autograd refuses to modify in place, and the projection's
            # backward needs its inputs, not this output.
            x2 = x.view(-1, x.shape[-1])
            _rope_launch(x2, x2, cos, sin, positions, nheads, head_dim, False)
            return torch.empty(0, dtype=x.dtype, device=x.device).set_(x.untyped_storage(), x.storage_offset(),
                                                                       x.shape, x.stride())
        src = x.reshape(-1, x.shape[-1])
        src = src if src.stride(-1) == 1 else src.contiguous()
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        _rope_launch(out.view(-1, out.shape[-1]), src, cos, sin, positions, nheads, head_dim, False)
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin, positions = ctx.saved_tensors
        nheads, head_dim, inplace = ctx.cfg
        if inplace and dy.is_contiguous():
            # the incoming gradient is a temporary of the attention backward: rotate it back in place
            d2 = dy.view(-1, dy.shape[-1])
            _rope_launch(d2, d2, cos, sin, positions, nheads, head_dim, True)
            return dy, None, None, None, None, None, None
        src = dy.reshape(-1, dy.shape[-1])
        src = src if src.stride(-1) == 1 else src.contiguous()
        dx = torch.empty(dy.shape, dtype=dy.dtype, device=dy.device)
        _rope_launch(dx.view(-1, dx.shape[-1]), src, cos, sin, positions, nheads, head_dim, True)
        return dx, None, None, None, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, nheads: int, head_dim: int,
         positions: Optional[torch.Tensor] = None, inplace: bool = False) -> torch.Tensor:
    """Rotate the first ``nheads`` heads of the last dim of ``x`` ([..., W], W >= nheads*head_dim).

    ``inplace``: overwrite ``x`` (and, in the backward pass, the incoming gradient) instead of writing a new
    tensor; only for an ``x`` that nothing else reads in its unrotated form, e.g. the output of the fused
    q|k|v projection. The columns that are not rotated then cost no memory traffic.

    Used on the fused q|k|v projection output: passing ``nheads = n_q + n_kv`` rotates q and k and
    leaves v untouched. Token position = ``positions`` (int32, one per row) or row index mod S.
    """
    if not (_lib.use_kernels(x, cos) and x.dtype == torch.bfloat16 and head_dim % 16 == 0 and x.shape[-1] % 8 == 0):
        return _RopeRef.apply(x, cos, sin, positions, nheads, head_dim)
    if positions is not None and positions.dtype != torch.int32:
        positions = positions.to(torch.int32)
    return _Rope.apply(x, cos, sin, positions, nheads, head_dim, bool(inplace) and not x.is_leaf)


class _RopeRef(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, positions, nheads, head_dim):
        ctx.save_for_backward(cos, sin, positions)
        ctx.cfg = (nheads, head_dim)
        return rope_reference(x, cos, sin, nheads, head_dim, positions, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin, positions = ctx.saved_tensors
        nheads, head_dim = ctx.cfg
        return rope_reference(dy, cos, sin, nheads, head_dim, positions, True), None, None, None, None, None


def swiglu_reference(gate_up: torch.Tensor) -> torch.Tensor:
    F = gate_up.shape[-1] // 2
    g, u = gate_up[..., :F].float(), gate_up[..., F:].float()
    return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        shp = gu.shape
        F = shp[-1] // 2
        gu2 = gu.reshape(-1, shp[-1])
        gu2 = gu2 if gu2.stride(-1) == 1 else gu2.contiguous()
        out = torch.empty(gu2.shape[0], F, dtype=gu.dtype, device=gu.device)
        rc = _lib.lib().atb_swiglu_fwd(_lib.ptr(gu2), _lib.ptr(out), ctypes.c_longlong(gu2.shape[0]), ctypes.c_int(F),
                                       ctypes.c_longlong(gu2.stride(0)), ctypes.c_longlong(F), _lib.stream_ptr())
        _lib.check(rc, "atb_swiglu_fwd")
        ctx.save_for_backward(gu2)
        ctx.shp = shp
        return out.view(*shp[:-1], F)

    @staticmethod
    def backward(ctx, dout):
        (gu2,) = ctx.saved_tensors
        return swiglu_backward(gu2, dout.reshape(-1, gu2.shape[1] // 2)).view(ctx.shp)


def swiglu_backward(gu2: torch.Tensor, d2: torch.Tensor) -> torch.Tensor:
    """Gradient of ``silu(gate) * up`` with respect to the fused ``[T, 2F]`` gate|up tensor (kernel launch)."""
    F = gu2.shape[1] // 2
    d2 = d2 if d2.is_contiguous() else d2.contiguous()
    dgu = torch.empty(gu2.shape[0], 2 * F, dtype=gu2.dtype, device=gu2.device)
    # dgu is written with the pitch of gu2; a contiguous gu2 is the common case
    src = gu2 if gu2.is_contiguous() else gu2.contiguous()
    rc = _lib.lib().atb_swiglu_bwd(_lib.ptr(src), _lib.ptr(d2), _lib.ptr(dgu), ctypes.c_longlong(src.shape[0]),
                                   ctypes.c_int(F), ctypes.c_longlong(2 * F), ctypes.c_longlong(F),
                                   _lib.stream_ptr())
    _lib.check(rc, "atb_swiglu_bwd")
    return dgu


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for a fused ``[..., 2F]`` gate|up tensor."""
    if not (_lib.use_kernels(gate_up) and gate_up.dtype == torch.bfloat16 and gate_up.shape[-1] % 16 == 0):
        return swiglu_reference(gate_up)
    return _SwiGLU.apply(gate_up)


def bias_gather_add_reference(inp, bias, expert_idx):
    return inp + bias[expert_idx.long()]


class _BiasGatherAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, bias, expert_idx):
        out = torch.empty_like(inp)
        idx = expert_idx.to(torch.int32)
        rc = _lib.lib().atb_bias_gather_add(_lib.ptr(inp), _lib.ptr(bias), _lib.ptr(idx), _lib.ptr(out),
                                            ctypes.c_longlong(inp.shape[0]), ctypes.c_int(inp.shape[1]),
                                            _lib.stream_ptr())
        _lib.check(rc, "atb_bias_gather_add")
        ctx.save_for_backward(idx)
        ctx.E = bias.shape[0]
        return out

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        # deterministic: segment sums in index order, fp32 accumulation
        db = torch.zeros(ctx.E, dy.shape[1], dtype=torch.float32, device=dy.device)
        db.index_add_(0, idx.long(), dy.float())
        return dy, db.to(dy.dtype), None


def bias_gather_add(inp: torch.Tensor, bias: torch.Tensor, expert_idx: torch.Tensor) -> torch.Tensor:
    """``out[t] = inp[t] + bias[expert_idx[t]]`` (per-expert bias of an MoE layer)."""
    if not (_lib.use_kernels(inp, bias) and inp.dtype == torch.bfloat16 and inp.dim() == 2 and inp.shape[1] % 8 == 0
            and inp.is_contiguous() and bias.is_contiguous() and bias.dtype == inp.dtype):
        return bias_gather_add_reference(inp, bias, expert_idx)
    return _BiasGatherAdd.apply(inp, bias, expert_idx)
