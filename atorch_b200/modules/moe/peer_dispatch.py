"""Expert-parallel token exchange over NVLink peer memory (``token_dispatcher_type="PeerMemory"``).

The all-to-all of an expert-parallel MoE layer without a collective call or a host sync (kernels in
csrc/moe.cu): the router's expert ids are turned into slot numbers on the device, every token row is
stored straight into the owning rank's expert buffer, the expert MLP runs as grouped GEMMs that read the
fill counts from device memory (empty tiles are skipped: ``ops.gemm(groups=...)``), and every rank pulls
its tokens' results back out of the owners' output buffers with the routing probabilities applied.
Capacity-factor routing: a (rank, expert) pair sends at most ``capacity`` tokens, later ones are dropped
(their contribution is zero), as in the reference's ``TopkGate`` capacity handling
(atorch/modules/moe/topk_gating.py:11-96); all shapes are static.

Each layer owns four symmetric buffers ``[E_local, W, capacity, H]`` (tokens in, expert outputs, and the
two gradient buffers of the backward pass), each with a signal pad:

    forward   scatter x -> X (peers)  | ARRIVE | zero unused slots | grouped MLP | Y | ARRIVE | gather Y (peers)
    backward  scatter p*dy -> GY, dp = <dy, Y rows> | ... | grouped MLP backward | GX | gather GX (peers)

Replaces ``MoEAllToAllTokenDispatcher`` + ``grouped_gemm`` on one NVSwitch domain (reference:
atorch/modules/moe/token_dispatcher.py:297-470, grouped_gemm_moe.py:816-879).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ... import _lib, ops
from ...parallel import symm
from ...parallel.symm import CH_ARRIVE, CH_DONE, CH_READY, SymmetricBuffer


def available(group) -> bool:
    if not symm.available():
        return False
    L = _lib.lib()
    return L is not None and L.has("atb_moe_scatter") and 1 <= dist.get_world_size(group) <= 8


def expert_capacity(tokens: int, topk: int, num_experts: int, capacity_factor: float) -> int:
    """Slots per (source rank, expert), rounded up to the 256-row tile of the grouped GEMM."""
    cap = math.ceil(capacity_factor * tokens * topk / num_experts)
    return max(256, (cap + 255) // 256 * 256)


class PeerExpertBuffers:
    """The symmetric buffers of one MoE layer (allocated on first use, sized for a fixed token count)."""

    def __init__(self, group, e_local: int, capacity: int, hidden: int, device):
        self.group, self.e_local, self.capacity, self.hidden = group, e_local, capacity, hidden
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.groups = e_local * self.world
        n = self.groups * capacity * hidden
        mk = lambda: SymmetricBuffer(n, torch.bfloat16, group, device)
        self.X, self.Y, self.GY, self.GX = mk(), mk(), mk(), mk()
        self.counts = SymmetricBuffer(max(64, self.groups), torch.int32, group, device)
        self.counts.tensor.zero_()
        self._count_ptrs = self.counts._data_ptrs

    def view(self, buf: SymmetricBuffer) -> torch.Tensor:
        return buf.tensor.view(self.groups * self.capacity, self.hidden)

    def local_counts(self) -> torch.Tensor:
        return self.counts.tensor[: self.groups]


def _i64(t: torch.Tensor) -> int:
    assert t.dtype in (torch.int64, torch.int32)
    return int(t.dtype == torch.int64)


def route(idx: torch.Tensor, num_experts: int, capacity: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Slot number of every routed entry (-1 = dropped) and the per-expert counts, on the device."""
    flat = idx.reshape(-1).contiguous()
    slot = torch.empty(flat.numel(), dtype=torch.int32, device=idx.device)
    count = torch.empty(num_experts, dtype=torch.int32, device=idx.device)
    rc = _lib.lib().atb_moe_route(_lib.ptr(flat), ctypes.c_int(_i64(flat)), ctypes.c_int(flat.numel()),
                                  ctypes.c_int(num_experts), ctypes.c_int(capacity), _lib.ptr(slot), _lib.ptr(count),
                                  _lib.stream_ptr())
    _lib.check(rc, "atb_moe_route")
    return slot, count


def _scatter(bufs: PeerExpertBuffers, dst: SymmetricBuffer, src: torch.Tensor, idx, slot, w, count, topk: int) -> None:
    """Rows of ``src [T, H]`` into the owners' ``dst`` buffers; afterwards every rank's rows are in place."""
    if dst.seq > 0:
        dst.wait(CH_READY, dst.seq)            # the owners are done with the previous contents
    dst.seq += 1
    src = src if src.stride(-1) == 1 else src.contiguous()
    flat = idx.reshape(-1)
    rc = _lib.lib().atb_moe_scatter(
        dst._data_ptrs, bufs._count_ptrs, dst._pad_ptrs, _lib.ptr(dst.counter), ctypes.c_int(bufs.rank),
        ctypes.c_int(bufs.world), ctypes.c_uint(dst.seq), _lib.ptr(src), ctypes.c_longlong(src.stride(0)),
        _lib.ptr(flat), ctypes.c_int(_i64(flat)), _lib.ptr(slot), _lib.ptr(w), _lib.ptr(count),
        ctypes.c_int(flat.numel()), ctypes.c_int(topk), ctypes.c_int(bufs.hidden), ctypes.c_int(bufs.e_local),
        ctypes.c_int(bufs.capacity), ctypes.c_int(bufs.e_local * bufs.world), ctypes.c_int(0), _lib.stream_ptr())
    _lib.check(rc, "atb_moe_scatter")
    dst.wait(CH_ARRIVE, dst.seq)               # tokens and counts of every source rank have landed
    rc = _lib.lib().atb_moe_zero_tail(_lib.ptr(dst.tensor), _lib.ptr(bufs.local_counts()), ctypes.c_int(bufs.groups),
                                      ctypes.c_int(bufs.capacity), ctypes.c_int(bufs.hidden), _lib.stream_ptr())
    _lib.check(rc, "atb_moe_zero_tail")


def _take(bufs: PeerExpertBuffers, buf: SymmetricBuffer) -> torch.Tensor:
    """Private copy of the received rows; the buffer is then free for the next exchange."""
    out = bufs.view(buf).clone()
    buf.signal(CH_READY, buf.seq)
    return out


def _publish(bufs: PeerExpertBuffers, buf: SymmetricBuffer, rows: torch.Tensor) -> None:
    """Make ``rows [groups*capacity, H]`` this rank's copy of ``buf`` and tell every rank."""
    if buf.seq > 0:
        buf.wait(CH_DONE, buf.seq)             # the peers have finished reading the previous contents
    bufs.view(buf).copy_(rows)
    buf.seq += 1
    buf.signal(CH_ARRIVE, buf.seq)


def _gather(bufs: PeerExpertBuffers, buf: SymmetricBuffer, idx, slot, w, T: int, topk: int, want_out: bool = True,
            g: Optional[torch.Tensor] = None) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``out[t] = sum_j w * row`` pulled from the owners' copies of ``buf`` (and ``dw = <g[t], row>``)."""
    dev = slot.device
    out = torch.empty(T, bufs.hidden, dtype=torch.bfloat16, device=dev) if want_out else None
    dw = torch.empty(T * topk, dtype=torch.float32, device=dev) if g is not None else None
    if g is not None and g.stride(-1) != 1:
        g = g.contiguous()
    flat = idx.reshape(-1)
    rc = _lib.lib().atb_moe_gather(
        buf._data_ptrs, buf._pad_ptrs, _lib.ptr(buf.counter), ctypes.c_int(bufs.rank), ctypes.c_int(bufs.world),
        ctypes.c_uint(buf.seq), _lib.ptr(out), ctypes.c_longlong(bufs.hidden), _lib.ptr(flat),
        ctypes.c_int(_i64(flat)), _lib.ptr(slot), _lib.ptr(w), _lib.ptr(g),
        ctypes.c_longlong(g.stride(0) if g is not None else 0), _lib.ptr(dw), ctypes.c_int(T), ctypes.c_int(topk),
        ctypes.c_int(bufs.hidden), ctypes.c_int(bufs.e_local), ctypes.c_int(bufs.capacity), ctypes.c_int(0),
        _lib.stream_ptr(), _lib.ptr(_lib.status_word(dev)))
    _lib.check(rc, "atb_moe_gather")
    return out, dw


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, slot, count, bufs: PeerExpertBuffers, topk: int):
        _scatter(bufs, bufs.X, x, idx, slot, None, count, topk)
        ctx.bufs, ctx.topk, ctx.T = bufs, topk, x.shape[0]
        ctx.save_for_backward(idx, slot)
        # fill counts of the local groups, written by the source ranks together with their tokens; copied
        # before the buffer is released, because a fast peer may already start the next exchange
        local_counts = bufs.local_counts().clone()
        ctx.mark_non_differentiable(local_counts)
        return _take(bufs, bufs.X), local_counts

    @staticmethod
    def backward(ctx, g_rows, _g_counts):
        idx, slot = ctx.saved_tensors
        bufs = ctx.bufs
        _publish(bufs, bufs.GX, g_rows)
        dx, _ = _gather(bufs, bufs.GX, idx, slot, None, ctx.T, ctx.topk)
        return dx, None, None, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, probs, idx, slot, count, bufs: PeerExpertBuffers, topk: int):
        _publish(bufs, bufs.Y, rows)
        w = probs.reshape(-1).float().contiguous()
        out, _ = _gather(bufs, bufs.Y, idx, slot, w, probs.shape[0], topk)
        ctx.bufs, ctx.topk, ctx.pshape, ctx.pdtype = bufs, topk, probs.shape, probs.dtype
        ctx.save_for_backward(w, idx, slot, count)
        return out

    @staticmethod
    def backward(ctx, dout):
        w, idx, slot, count = ctx.saved_tensors
        bufs, topk = ctx.bufs, ctx.topk
        dout = dout.contiguous()
        # d prob = <dy[t], expert output row>: the owners' Y buffers still hold this layer's outputs
        _, dw = _gather(bufs, bufs.Y, idx, slot, None, dout.shape[0], topk, want_out=False, g=dout)
        # d rows = prob * dy[t], stored into the owners' gradient buffers
        _scatter(bufs, bufs.GY, dout, idx, slot, w, count, topk)
        g_rows = _take(bufs, bufs.GY)
        return g_rows, dw.view(ctx.pshape).to(ctx.pdtype), None, None, None, None, None


class _GroupedLinear(torch.autograd.Function):
    """``y[g] = x[g] W[e(g)]^T`` over the slot groups of an expert buffer. ``w`` is ``[E_local, N, K]``
    (``w_is_nk``) or ``[E_local, K, N]``; either way the GEMMs read it as stored."""

    @staticmethod
    def forward(ctx, x, w, counts, capacity: int, world: int, w_is_nk: bool):
        E = w.shape[0]
        grp = {"counts": counts, "m_rows": capacity}
        if E > 1:
            grp.update(n_b=E, bm_rows=world * capacity)
        y = ops.gemm(x, w.reshape(E * w.shape[1], w.shape[2]), b_mn=not w_is_nk, groups=grp)
        ctx.save_for_backward(x, w, counts)
        ctx.cfg = (capacity, world, w_is_nk)
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, counts = ctx.saved_tensors
        capacity, world, w_is_nk = ctx.cfg
        E = w.shape[0]
        dy = dy.contiguous()
        grp = {"counts": counts, "m_rows": capacity}
        if E > 1:
            grp.update(n_b=E, bm_rows=world * capacity)
        # dx = dy W: the weight is the B operand again, in the other major-ness
        dx = ops.gemm(dy, w.reshape(E * w.shape[1], w.shape[2]), b_mn=w_is_nk, groups=grp)
        mg = getattr(ctx.w_ref, "main_grad", None)
        dw = mg if mg is not None else torch.empty_like(w)
        R = world * capacity
        for e in range(E):
            ge = {"counts": counts[e * world: (e + 1) * world], "k_rows": capacity}
            dye, xe = dy[e * R: (e + 1) * R], x[e * R: (e + 1) * R]
            if w_is_nk:      # dW[N, K] = dy^T x
                ops.gemm(dye, xe, a_mn=True, b_mn=True, out=dw[e], accumulate=mg is not None, groups=ge)
            else:            # dW[K, N] = x^T dy
                ops.gemm(xe, dye, a_mn=True, b_mn=True, out=dw[e], accumulate=mg is not None, groups=ge)
        if mg is not None:
            ctx.w_ref.grad_added_to_main_grad = True
            return dx, None, None, None, None, None
        return dx, dw, None, None, None, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, capacity: int, world: int,
                   w_is_nk: bool = True) -> torch.Tensor:
    return _GroupedLinear.apply(x, w, counts, capacity, world, w_is_nk)


class MoEPeerMemoryTokenDispatcher:
    """Interface of the token dispatchers of :mod:`token_dispatcher` on top of the peer-memory exchange."""

    def __init__(self, num_local_experts: int, local_expert_indices, num_experts: int, topk: int, ep_group=None,
                 use_expert_parallelism: bool = True, capacity_factor: float = 1.25):
        self.num_local_experts, self.num_experts, self.topk = num_local_experts, num_experts, topk
        self.ep_group = ep_group if ep_group is not None else dist.group.WORLD
        self.ep_size = dist.get_world_size(self.ep_group)
        self.capacity_factor = capacity_factor
        self.bufs: Optional[PeerExpertBuffers] = None

    def _buffers(self, tokens: int, hidden: int, device) -> PeerExpertBuffers:
        cap = expert_capacity(tokens, self.topk, self.num_experts, self.capacity_factor)
        b = self.bufs
        if b is None or b.capacity != cap or b.hidden != hidden:
            self.bufs = b = PeerExpertBuffers(self.ep_group, self.num_local_experts, cap, hidden, device)
        return b

    def token_permutation(self, hidden_states, probs, indices, se_fn1=None):
        self.hidden_shape = hidden_states.shape
        x = hidden_states.reshape(-1, hidden_states.shape[-1])
        if x.dtype != torch.bfloat16:
            raise TypeError("the peer-memory dispatcher exchanges bf16 rows")
        bufs = self._buffers(x.shape[0], x.shape[1], x.device)
        self.indices = indices.reshape(x.shape[0], -1)
        self.probs = probs
        self.slot, self.count = route(self.indices, self.num_experts, bufs.capacity)
        rows, self.local_counts = _Dispatch.apply(x, self.indices, self.slot, self.count, bufs, self.topk)
        se_out = se_fn1(hidden_states) if se_fn1 is not None else None
        return rows, self.local_counts, se_out

    def token_unpermutation(self, expert_output, se_fn2=None, se_fn2_additional_input=None):
        out = _Combine.apply(expert_output, self.probs, self.indices, self.slot, self.count, self.bufs, self.topk)
        se_out = None
        if se_fn2 is not None:
            se_out = se_fn2(*se_fn2_additional_input) if isinstance(se_fn2_additional_input, (tuple, list)) \
                else se_fn2(se_fn2_additional_input)
        return out.view(self.hidden_shape), se_out
