"""Ring (context-parallel) attention on the flash kernels, with the key/value exchange over peer memory.

Every rank of the sequence-parallel group holds ``S / W`` tokens of q, k and v (contiguous chunks in rank order).
Forward on rank r: its k|v chunk is published in a symmetric buffer; the copy engines pull the peers' chunks one
after the other into two local staging buffers (a chunk crosses NVLink once, while the previous chunk is being
processed), the flash forward kernel runs per chunk and returns ``(out_i, lse_i)``, and the partial results are
merged with the log-sum-exp rule. With a causal mask only the chunks of ranks <= r are visited and the own chunk
is the only one that needs the causal form.

Backward: with the final ``out`` and ``lse`` the flash backward kernels give the exact contribution of every
chunk (``P = exp(S - lse)`` is already globally normalised): ``dq`` accumulates locally, the ``dk | dv`` of a
remote chunk is added (fp32 ``red.add`` through NVLink) into its owner's symmetric accumulation buffer.

The reference has no ring attention of its own (it reaches context parallelism only through Megatron); the
sequence-parallel hook it does have is ``seq_all_to_all`` (atorch/distributed/distributed.py:613-679).
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, Tuple

import torch
import torch.distributed as dist

from .. import _lib
from . import flash


def available(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group) -> bool:
    from ..parallel import symm

    if not (q.is_cuda and symm.available() and flash.supported(q, k, v) and flash.backward_built()):
        return False
    L = _lib.lib()
    W = dist.get_world_size(group)
    return L.has("atb_peer_add_bf16") and 1 < W <= 8 and k.shape == v.shape and k.numel() % 8 == 0


class _Ctx:
    """Buffers of one (group, k|v chunk shape): the published chunk, two staging buffers, the fp32 gradient
    accumulator that the peers add into."""

    def __init__(self, group, shape: Tuple[int, ...], device):
        from ..parallel.symm import SymmetricBuffer

        self.group, self.shape = group, shape
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        n = 2 * math.prod(shape)
        self.n = n
        self.kv = SymmetricBuffer(n, torch.bfloat16, group, device)
        self.acc = SymmetricBuffer(n, torch.float32, group, device)
        self.acc.tensor.zero_()
        self.stage = [torch.empty(n, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.copy_stream = torch.cuda.Stream(device)
        self.acc_ptrs = [int(p) for p in self.acc._data_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group=group)


_ctxs: Dict[Tuple, _Ctx] = {}


def _ctx(group, shape, device) -> _Ctx:
    key = (id(group), tuple(shape), device.index)
    c = _ctxs.get(key)
    if c is None:
        c = _ctxs[key] = _Ctx(group, tuple(shape), device)
    return c


def _visit_chunks(c: _Ctx, k: torch.Tensor, v: torch.Tensor, causal: bool, fn) -> None:
    """Publish this rank's k|v, then call ``fn(owner_rank, k_chunk, v_chunk, is_own)`` for the own chunk and for
    every peer chunk this rank needs, with the next chunk's copy in flight while ``fn`` works on the current one."""
    from ..parallel.symm import CH_DONE, CH_READY

    W, r, half = c.world, c.rank, c.n // 2
    dev = k.device
    cur = torch.cuda.current_stream(dev)
    if c.kv.seq > 0:
        c.kv.wait(CH_DONE, c.kv.seq)              # every peer has finished pulling the previous contents
    c.kv.tensor[:half].copy_(k.reshape(-1))
    c.kv.tensor[half:].copy_(v.reshape(-1))
    c.kv.seq += 1
    c.kv.signal(CH_READY, c.kv.seq)
    peers = [(r - s) % W for s in range(1, W)]
    if causal:
        peers = [p for p in peers if p < r]       # later chunks of the sequence are invisible to this rank's queries
    copied, done = {}, {}
    c.copy_stream.wait_stream(cur)
    with torch.cuda.stream(c.copy_stream):
        c.kv.wait(CH_READY, c.kv.seq)             # every rank's chunk is published

    def start_copy(i: int) -> None:
        with torch.cuda.stream(c.copy_stream):
            if i >= 2:
                c.copy_stream.wait_event(done[i - 2])          # the staging buffer's previous chunk has been used
            c.stage[i % 2].copy_(c.kv.peer_view(peers[i]), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(c.copy_stream)
            copied[i] = ev

    if peers:
        start_copy(0)
    fn(r, k, v, True)
    for i, p in enumerate(peers):
        if i + 1 < len(peers):
            start_copy(i + 1)
        cur.wait_event(copied[i])
        st = c.stage[i % 2]
        fn(p, st[:half].view(c.shape), st[half:].view(c.shape), False)
        ev = torch.cuda.Event()
        ev.record(cur)
        done[i] = ev
    with torch.cuda.stream(c.copy_stream):
        c.kv.signal(CH_DONE, c.kv.seq)            # after this rank's last pull
    for t in c.stage:
        t.record_stream(c.copy_stream)


def zigzag_shard(x: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """This rank's part of ``x`` in the load-balanced layout for causal ring attention: the sequence is cut into
    ``2 W`` pieces and rank r holds pieces ``r`` and ``2 W - 1 - r`` (in that order)."""
    pieces = x.chunk(2 * world, dim)
    return torch.cat([pieces[rank], pieces[2 * world - 1 - rank]], dim)


def zigzag_unshard(parts, dim: int = 1) -> torch.Tensor:
    """Inverse of ``zigzag_shard`` for the list of all ranks' parts."""
    world = len(parts)
    lo = [p.chunk(2, dim)[0] for p in parts]
    hi = [p.chunk(2, dim)[1] for p in parts]
    return torch.cat(lo + hi[::-1], dim)


def _plan(owner: int, rank: int, causal: bool, zigzag: bool, S: int):
    """Which (query rows, key rows, causal?) products this rank computes against ``owner``'s chunk. Contiguous
    layout: everything against an earlier (or, without a mask, any) chunk. Zigzag layout with a causal mask: both
    query halves against the first key half of an earlier rank, the second query half against both key halves of a
    later rank - two half-by-half products per peer on every rank."""
    full = slice(0, S)
    if owner == rank:
        return [(full, full, causal)]
    if not (causal and zigzag):
        return [(full, full, False)]
    h = S // 2
    return [(full, slice(0, h), False)] if owner < rank else [(slice(h, S), full, False)]


class _RingFlash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, causal, scale, zigzag):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        c = _ctx(group, k.shape, k.device)
        B, S, H, _ = q.shape
        out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        lse = torch.full((B, H, S), float("-inf"), dtype=torch.float32, device=q.device)

        def step(owner, kc, vc, is_own):
            for qs, ks, cz in _plan(owner, c.rank, causal, zigzag, S):
                whole_q = qs.stop - qs.start == S
                qq = q if whole_q else q[:, qs].contiguous()
                kk, vv = (kc, vc) if ks.stop - ks.start == S else (kc[:, ks].contiguous(), vc[:, ks].contiguous())
                o_i, lse_i = flash.flash_fwd_raw(qq, kk, vv, cz, scale, None, None)
                old = lse[:, :, qs]
                new = torch.logaddexp(old, lse_i)                            # [B, H, rows]; the own chunk comes first,
                w_old = torch.exp(old - new).transpose(1, 2).unsqueeze(-1)   # so `new` is finite from then on
                w_new = torch.exp(lse_i - new).transpose(1, 2).unsqueeze(-1)
                out[:, qs] = out[:, qs] * w_old + o_i.float() * w_new
                lse[:, :, qs] = new

        _visit_chunks(c, k, v, causal and not zigzag, step)
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (group, causal, scale, zigzag)
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..parallel.symm import CH_ARRIVE, CH_READY

        q, k, v, out, lse = ctx.saved_tensors
        group, causal, scale, zigzag = ctx.cfg
        S = q.shape[1]
        c = _ctx(group, k.shape, k.device)
        dout = dout.contiguous()
        if c.acc.seq > 0:
            c.acc.wait(CH_READY, c.acc.seq)          # every owner has taken (and zeroed) its previous sums
        c.acc.seq += 1
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        keep = []

        def step(owner, kc, vc, is_own):
            for qs, ks, cz in _plan(owner, c.rank, causal, zigzag, S):
                whole_q, whole_k = qs.stop - qs.start == S, ks.stop - ks.start == S
                sub = (lambda t: t) if whole_q else (lambda t: t[:, qs].contiguous())
                kk, vv = (kc, vc) if whole_k else (kc[:, ks].contiguous(), vc[:, ks].contiguous())
                lse_q = lse if whole_q else lse[:, :, qs].contiguous()
                dq_i, dk_i, dv_i = flash.flash_bwd_raw(sub(dout), sub(q), kk, vv, sub(out), lse_q, cz, scale, None, None)
                dq[:, qs] += dq_i
                if whole_k:
                    dkv = torch.cat([dk_i.reshape(-1), dv_i.reshape(-1)])
                else:                        # a key half: the other half of the owner's gradient gets zeros
                    full = torch.zeros((2,) + tuple(kc.shape), dtype=dk_i.dtype, device=dk_i.device)
                    full[0][:, ks] = dk_i
                    full[1][:, ks] = dv_i
                    dkv = full.reshape(-1)
                rc = _lib.lib().atb_peer_add_bf16(ctypes.c_ulonglong(c.acc_ptrs[owner]), _lib.ptr(dkv),
                                                  ctypes.c_longlong(dkv.numel()), _lib.stream_ptr())
                _lib.check(rc, "atb_peer_add_bf16")
                keep.append(dkv)

        _visit_chunks(c, k, v, causal and not zigzag, step)
        c.acc.signal(CH_ARRIVE, c.acc.seq)           # my contributions are out
        c.acc.wait(CH_ARRIVE, c.acc.seq)             # ... and everybody's are in
        half = c.n // 2
        dk = c.acc.tensor[:half].view(k.shape).to(k.dtype)
        dv = c.acc.tensor[half:].view(v.shape).to(v.dtype)
        c.acc.tensor.zero_()
        c.acc.signal(CH_READY, c.acc.seq)
        return dq.to(q.dtype), dk, dv, None, None, None, None


def ring_flash_attention(q, k, v, group, causal: bool = True, softmax_scale=None, layout: str = "contiguous"):
    """q, k, v: this rank's ``[B, S / W, H, D]`` part of the sequence; returns the attention output of the local
    queries over the whole sequence. ``layout="contiguous"``: parts are consecutive chunks in rank order (with a
    causal mask rank r then works on r + 1 chunks). ``layout="zigzag"``: parts made by ``zigzag_shard`` (pieces r
    and 2 W - 1 - r), which gives every rank the same amount of causal work."""
    assert layout in ("contiguous", "zigzag"), layout
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
    zigzag = layout == "zigzag" and causal
    assert not zigzag or q.shape[1] % 2 == 0
    return _RingFlash.apply(q, k, v, group, bool(causal), float(scale), zigzag)
