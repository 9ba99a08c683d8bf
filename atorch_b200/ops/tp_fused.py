"""Tensor-parallel linears with sequence-sharded activations, fused with their collectives over NVLink.

Megatron-style sequence parallelism keeps the activations between the tensor-parallel blocks sharded along
the sequence: a column-parallel linear starts with an all-gather of its input, a row-parallel linear ends
with a reduce-scatter of its output. Here both are one GEMM launch each (csrc/gemm_bf16_2cta.cu):

``allgather_linear(x_local, w)``   ``y[S, N] = all_gather(x)[S, K] @ w[N, K]^T``. The local shard goes into a
    symmetric buffer, the copy engines pull the peers' shards into a full ``[S, K]`` buffer and raise one
    arrival flag per shard; the GEMM is launched at once, visits the tiles of this rank's own shard first and
    its TMA producer waits (bounded) on the flag of the shard a tile needs - transfers hide behind the math.
``linear_reduce_scatter(x, w)``    ``y_local[S/W, N] = reduce_scatter(x[S, K] @ w[N, K]^T)``. The GEMM
    epilogue adds every output row, as fp32 ``red.add`` on peer pointers, into the accumulation buffer of the
    rank that owns the row: no partial-sum tensor, no separate collective.

Each is the other's backward: d(all-gather -> GEMM)/dx is a GEMM -> reduce-scatter and vice versa, so the
autograd functions below call each other's kernels. Used by ``ColumnParallelLinear`` /
``RowParallelLinear(sequence_parallel=True)`` on 2..8 GPUs of one NVSwitch domain; elsewhere those layers
use ``torch.distributed`` collectives around ``ops.linear``.
(The reference reaches sequence-parallel linears only through Megatron; its own layers are all-reduce style:
atorch/modules/distributed_modules/layers.py:373-389,531-546.)
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _lib
from .gemm import gemm


def available(group) -> bool:
    from ..parallel import symm

    if not symm.available():
        return False
    L = _lib.lib()
    return L is not None and L.has("atb_gemm_bf16_2cta_fused") and 1 < dist.get_world_size(group) <= 8


def shapes_ok(rows_local: int, n: int, k: int) -> bool:
    """The fused kernels need whole 256-row tiles per shard and 8-element aligned feature dims."""
    return rows_local % 256 == 0 and n % 8 == 0 and k % 8 == 0 and n >= 256


class _Context:
    """Symmetric buffers of one (group, shard shape): shared by all layers with that shape; the flag
    protocol serialises their uses."""

    def __init__(self, group, rows: int, feat: int, device):
        from ..parallel.symm import SymmetricBuffer

        self.group, self.rows, self.feat = group, rows, feat
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.x = SymmetricBuffer(rows * feat, torch.bfloat16, group, device)      # this rank's shard, for the peers
        self.acc = SymmetricBuffer(rows * feat, torch.float32, group, device)     # reduce-scatter accumulation
        self.acc.tensor.zero_()
        self.flags = torch.zeros(self.world, dtype=torch.int32, device=device)
        self.epoch = 0
        self.copy_stream = torch.cuda.Stream(device)
        self._acc_ptrs = self.acc._data_ptrs
        torch.cuda.synchronize(device)
        dist.barrier(group=group)


_contexts: Dict[Tuple, _Context] = {}


def _ctx(group, rows: int, feat: int, device) -> _Context:
    key = (id(group), rows, feat, device.index)
    c = _contexts.get(key)
    if c is None:
        c = _contexts[key] = _Context(group, rows, feat, device)
    return c


def _ag_gemm(x_local: torch.Tensor, b: torch.Tensor, b_mn: bool, group) -> Tuple[torch.Tensor, torch.Tensor]:
    """``all_gather(x_local)[S, K] @ op(b)`` -> (y [S, N], gathered x [S, K])."""
    from ..parallel.symm import CH_DONE, CH_READY

    rows, K = x_local.shape
    c = _ctx(group, rows, K, x_local.device)
    W, r = c.world, c.rank
    N = b.shape[1] if b_mn else b.shape[0]
    cur = torch.cuda.current_stream(x_local.device)
    # 1. publish this rank's shard (after every rank has finished pulling the previous one)
    if c.x.seq > 0:
        c.x.wait(CH_DONE, c.x.seq)
    c.x.tensor.view(rows, K).copy_(x_local)
    c.x.seq += 1
    c.x.signal(CH_READY, c.x.seq)
    # 2. copy engines: own shard first, then the peers' (each after its READY), one arrival flag per shard
    x_full = torch.empty(W * rows, K, dtype=torch.bfloat16, device=x_local.device)
    c.epoch += 1
    c.copy_stream.wait_stream(cur)
    with torch.cuda.stream(c.copy_stream):
        x_full[r * rows: (r + 1) * rows].copy_(c.x.tensor.view(rows, K))
        c.flags[r: r + 1].fill_(c.epoch)
        c.x.wait(CH_READY, c.x.seq)
        for k in range(1, W):
            p = (r + k) % W
            x_full[p * rows: (p + 1) * rows].copy_(c.x.peer_view(p).view(rows, K), non_blocking=True)
            c.flags[p: p + 1].fill_(c.epoch)
        c.x.signal(CH_DONE, c.x.seq)
        ev = torch.cuda.Event()
        ev.record(c.copy_stream)
    x_full.record_stream(c.copy_stream)
    # 3. the GEMM starts right away and follows the flags
    y = torch.empty(W * rows, N, dtype=torch.bfloat16, device=x_local.device)
    rc = _lib.lib().atb_gemm_bf16_2cta_fused(
        _lib.ptr(x_full), _lib.ptr(b), _lib.ptr(y), ctypes.c_int(W * rows), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_longlong(K), ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(N), ctypes.c_int(0),
        ctypes.c_int(int(b_mn)), ctypes.c_float(1.0), _lib.ptr(c.flags), ctypes.c_uint(c.epoch), ctypes.c_int(rows),
        ctypes.c_int(r * rows), None, ctypes.c_int(0), ctypes.c_int(0), _lib.stream_ptr(),
        _lib.ptr(_lib.status_word(x_local.device)))
    _lib.check(rc, "atb_gemm_bf16_2cta_fused (all-gather -> GEMM)")
    cur.wait_event(ev)            # later users of the gathered tensor need all of it
    return y, x_full


def _gemm_rs(a: torch.Tensor, b: torch.Tensor, b_mn: bool, group, a_mn: bool = False,
             out_dtype=torch.bfloat16) -> torch.Tensor:
    """``reduce_scatter(op(a)[S, K] @ op(b))`` -> y_local [S/W, N]; ``a_mn``: a is stored ``[K, S]``."""
    from ..parallel.symm import CH_ARRIVE, CH_READY

    K, S = a.shape if a_mn else a.shape[::-1]
    N = b.shape[1] if b_mn else b.shape[0]
    W = dist.get_world_size(group)
    rows = S // W
    c = _ctx(group, rows, N, a.device)
    if c.acc.seq > 0:
        c.acc.wait(CH_READY, c.acc.seq)      # every owner has taken (and zeroed) its previous sums
    c.acc.seq += 1
    a = a if a.stride(-1) == 1 else a.contiguous()
    rc = _lib.lib().atb_gemm_bf16_2cta_fused(
        _lib.ptr(a), _lib.ptr(b), None, ctypes.c_int(S), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(N),
        ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)), ctypes.c_float(1.0), None, ctypes.c_uint(0), ctypes.c_int(0),
        ctypes.c_int(0), c._acc_ptrs, ctypes.c_int(W), ctypes.c_int(rows), _lib.stream_ptr(), _lib.ptr(_lib.status_word(a.device)))
    _lib.check(rc, "atb_gemm_bf16_2cta_fused (GEMM -> reduce-scatter)")
    c.acc.signal(CH_ARRIVE, c.acc.seq)       # my contributions are out
    c.acc.wait(CH_ARRIVE, c.acc.seq)         # ... and everybody's are in
    y = c.acc.tensor.view(rows, N).to(out_dtype, copy=True)
    c.acc.tensor.zero_()
    c.acc.signal(CH_READY, c.acc.seq)
    return y


class _AllGatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight, group):
        y, x_full = _ag_gemm(x_local, weight, False, group)
        ctx.save_for_backward(x_full, weight)
        ctx.group, ctx.w_ref = group, weight
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx_local = _gemm_rs(dy, weight, True, ctx.group) if ctx.needs_input_grad[0] else None   # (dy W) reduce-scattered
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                first = getattr(ctx.w_ref, "_atb_first", False)
                gemm(dy, x_full, a_mn=True, b_mn=True, out=mg, accumulate=not first)
                ctx.w_ref._atb_first = False
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                dw = gemm(dy, x_full, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        return dx_local, dw, None


class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, group):
        y_local = _gemm_rs(x, weight, False, group)
        ctx.save_for_backward(x, weight)
        ctx.group, ctx.w_ref = group, weight
        return y_local

    @staticmethod
    def backward(ctx, dy_local):
        x, weight = ctx.saved_tensors
        dy_local = dy_local.contiguous()
        # dx = all_gather(dy) W ; the gathered dy also feeds the weight gradient
        dx, dy_full = _ag_gemm(dy_local, weight, True, ctx.group)
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                first = getattr(ctx.w_ref, "_atb_first", False)
                gemm(dy_full, x, a_mn=True, b_mn=True, out=mg, accumulate=not first)
                ctx.w_ref._atb_first = False
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                dw = gemm(dy_full, x, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        return (dx if ctx.needs_input_grad[0] else None), dw, None


def allgather_linear(x_local: torch.Tensor, weight: torch.Tensor, group) -> torch.Tensor:
    """``all_gather(x_local, dim=-2) @ weight^T`` with ``x_local [..., S/W, K]`` (leading dims of size 1)."""
    lead = x_local.shape[:-2]
    x2 = x_local.reshape(-1, x_local.shape[-1])
    y = _AllGatherLinear.apply(x2 if x2.stride(-1) == 1 else x2.contiguous(), weight, group)
    return y.view(*lead, y.shape[0], y.shape[1])


def linear_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, group) -> torch.Tensor:
    """``reduce_scatter(x @ weight^T, dim=-2)`` with ``x [..., S, K]`` (leading dims of size 1)."""
    lead = x.shape[:-2]
    x2 = x.reshape(-1, x.shape[-1])
    y = _LinearReduceScatter.apply(x2, weight, group)
    return y.view(*lead, y.shape[0], y.shape[1])


# ------------------------------------------------------------------------------------------------------
# Row-sharded weight (per-parameter ZeRO-3 / FSDP sharding along dim 0): the all-gather of the weight is fused
# into the GEMM that consumes it, the reduce-scatter of its gradient into the GEMM that produces it.
# ------------------------------------------------------------------------------------------------------
def _gather_rows(w_shard: torch.Tensor, group, wait: bool):
    """Copy-engine all-gather of ``w_shard [N/W, K]`` into a full ``[N, K]`` tensor, one arrival flag per shard.
    Returns (w_full, context, event); with ``wait`` the current stream waits for all shards."""
    from ..parallel.symm import CH_DONE, CH_READY

    rows, K = w_shard.shape
    c = _ctx(group, rows, K, w_shard.device)
    W, r = c.world, c.rank
    cur = torch.cuda.current_stream(w_shard.device)
    if c.x.seq > 0:
        c.x.wait(CH_DONE, c.x.seq)
    c.x.tensor.view(rows, K).copy_(w_shard)
    c.x.seq += 1
    c.x.signal(CH_READY, c.x.seq)
    w_full = torch.empty(W * rows, K, dtype=torch.bfloat16, device=w_shard.device)
    c.epoch += 1
    c.copy_stream.wait_stream(cur)
    with torch.cuda.stream(c.copy_stream):
        w_full[r * rows: (r + 1) * rows].copy_(c.x.tensor.view(rows, K))
        c.flags[r: r + 1].fill_(c.epoch)
        c.x.wait(CH_READY, c.x.seq)
        for k in range(1, W):
            p = (r + k) % W
            w_full[p * rows: (p + 1) * rows].copy_(c.x.peer_view(p).view(rows, K), non_blocking=True)
            c.flags[p: p + 1].fill_(c.epoch)
        c.x.signal(CH_DONE, c.x.seq)
        ev = torch.cuda.Event()
        ev.record(c.copy_stream)
    w_full.record_stream(c.copy_stream)
    if wait:
        cur.wait_event(ev)
    return w_full, c, ev


class _ShardedWeightLinear(torch.autograd.Function):
    """``y = x @ all_gather(w_shard)^T``. Forward: the GEMM starts with this rank's own rows of the weight and its
    TMA producer waits (bounded) on the arrival flag of the shard a tile's weight rows come from. Backward: the
    weight is gathered again (it is not kept between the passes, as with reshard-after-forward), ``dx`` is a
    plain GEMM and the weight gradient ``dy^T x``, summed over the ranks, is added row by row into its owner's
    fp32 buffer by the GEMM epilogue, so each rank ends with the gradient of its own shard."""

    @staticmethod
    def forward(ctx, x, w_shard, group):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
        w_full, c, ev = _gather_rows(w_shard, group, wait=False)
        M, K = x2.shape
        N = w_full.shape[0]
        y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        rc = _lib.lib().atb_gemm_bf16_2cta_wgather(
            _lib.ptr(x2), _lib.ptr(w_full), _lib.ptr(y), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
            ctypes.c_longlong(x2.stride(0)), ctypes.c_longlong(K), ctypes.c_longlong(N), _lib.ptr(c.flags),
            ctypes.c_uint(c.epoch), ctypes.c_int(c.rows), ctypes.c_int(c.rank * c.rows), _lib.stream_ptr(),
            _lib.ptr(_lib.status_word(x.device)))
        _lib.check(rc, "atb_gemm_bf16_2cta_wgather (weight all-gather -> GEMM)")
        torch.cuda.current_stream(x.device).wait_event(ev)     # w_full is freed after this call
        ctx.save_for_backward(x2, w_shard)
        ctx.group, ctx.x_shape, ctx.w_ref = group, shp, w_shard
        return y.view(*shp[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, w_shard = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            w_full, _, _ = _gather_rows(w_shard, ctx.group, wait=True)
            dx = gemm(dy2, w_full, b_mn=True, out_dtype=x2.dtype).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            # dW [N, K] = dy^T x, reduce-scattered over its rows: both operands are read as stored
            g = _gemm_rs(dy2, x2, True, ctx.group, a_mn=True, out_dtype=torch.float32)
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                mg.add_(g) if mg.dtype == g.dtype else mg.add_(g.to(mg.dtype))
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                dw = g.to(w_shard.dtype)
        return dx, dw, None


def sharded_weight_available(group, rows_local: int, n_total: int, k: int) -> bool:
    L = _lib.lib()
    return (available(group) and L.has("atb_gemm_bf16_2cta_wgather") and rows_local % 256 == 0 and k % 8 == 0
            and n_total % 8 == 0)


def sharded_weight_linear(x: torch.Tensor, w_shard: torch.Tensor, group) -> torch.Tensor:
    """Linear layer whose weight ``[N, K]`` is sharded by rows over ``group`` (``w_shard [N/W, K]`` on each rank),
    every rank with its own ``x``: the data-parallel ZeRO-3 case. The weight gradient returned (or added to
    ``w_shard.main_grad``) is the SUM over the ranks of the gradient rows this rank owns."""
    W = dist.get_world_size(group)
    if x.dtype == torch.bfloat16 and w_shard.dtype == torch.bfloat16 and x.is_cuda and \
            sharded_weight_available(group, w_shard.shape[0], w_shard.shape[0] * W, w_shard.shape[1]):
        return _ShardedWeightLinear.apply(x, w_shard, group)
    return _ShardedWeightLinearRef.apply(x, w_shard, group)


class _ShardedWeightLinearRef(torch.autograd.Function):
    """The same contract with ``torch.distributed`` collectives around plain matmuls (CPU / gloo, odd shapes)."""

    @staticmethod
    def forward(ctx, x, w_shard, group):
        W = dist.get_world_size(group)
        parts = [torch.empty_like(w_shard) for _ in range(W)]
        dist.all_gather(parts, w_shard.contiguous(), group=group)
        w_full = torch.cat(parts, 0)
        ctx.save_for_backward(x, w_shard)
        ctx.group = group
        return x @ w_full.t()

    @staticmethod
    def backward(ctx, dy):
        x, w_shard = ctx.saved_tensors
        W = dist.get_world_size(ctx.group)
        parts = [torch.empty_like(w_shard) for _ in range(W)]
        dist.all_gather(parts, w_shard.contiguous(), group=ctx.group)
        w_full = torch.cat(parts, 0)
        dx = dy @ w_full
        dw_full = (dy.reshape(-1, dy.shape[-1]).float().t() @ x.reshape(-1, x.shape[-1]).float())
        dist.all_reduce(dw_full, group=ctx.group)
        r = dist.get_rank(ctx.group)
        rows = w_shard.shape[0]
        return dx, dw_full[r * rows: (r + 1) * rows].to(w_shard.dtype), None
