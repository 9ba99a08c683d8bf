"""Symmetric (peer-mapped) buffers and the fused collective kernels that run on them.

``SymmetricBuffer(numel, dtype, group)`` allocates the same buffer on every rank of ``group`` with
``torch.distributed._symmetric_memory`` (CUDA VMM + handle exchange), so every rank holds device
addresses of all peers' copies, a signal pad, and - on NVSwitch systems with NVLink SHARP - a multicast
address of the buffer. The methods launch the kernels of ``csrc/comm.cu``, which read the peers' data
over NVLink from inside the kernel that does the arithmetic (peer loads, or ``multimem.ld_reduce``
where the switch adds the ranks' values):

* ``reduce_scatter_into(out, ...)``       reduce-scatter into a local fp32 shard (optionally accumulating)
* ``reduce_scatter_adamw(...)``           gradient reduce-scatter fused with the sharded AdamW step
* ``all_reduce_(scale)``                  all-reduce in place
* ``allreduce_nesterov(...)``             local-SGD outer step (parameter mean + Nesterov + write-back)
* ``all_gather_into(out)``                pull every peer's buffer into a local tensor (SM kernel)
* ``copy_engine_all_gather(out, ...)``    the same on the copy engines: one peer copy per rank, no SM
  is used, so it overlaps compute kernels without slowing them (measured on B200: 721 GB/s per
  direction and no change in the time of concurrent GEMMs, against +100 % of its own duration for an
  NCCL all-gather kernel)
* ``signal(channel)`` / ``wait(channel)`` stream-ordered cross-rank flags

Each use of a buffer by a collective kernel has a sequence number (``seq``) that every rank counts the
same way; the kernels synchronise on ``slot >= seq`` in the signal pads. After a kernel that read the
peers' copies, ``wait_peers_done()`` must run on the stream that next overwrites the local copy. A wait
that runs out raises ``CommTimeoutError`` at the next ``check()``.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _lib

CH_ARRIVE, CH_MID, CH_DONE, CH_READY = 0, 1, 2, 3


class CommTimeoutError(RuntimeError):
    pass


def available() -> bool:
    if not (torch.cuda.is_available() and dist.is_available() and dist.is_initialized()):
        return False
    L = _lib.lib()
    return L is not None and L.has("atb_p2p_allreduce")


def nvls_wanted() -> bool:
    """Multimem kernels are used when the buffer has a multicast address, unless ATB_NVLS=0."""
    return os.environ.get("ATB_NVLS", "1") != "0"


def set_wait_limit_ns(ns: int) -> None:
    """Upper bound of the cross-rank waits of kernels launched from now on (default 2 s)."""
    _lib.check(_lib.lib().atb_set_comm_wait_ns(ctypes.c_ulonglong(int(ns))), "atb_set_comm_wait_ns")


class SymmetricBuffer:
    MAX_RANKS = 8

    def __init__(self, numel: int, dtype: torch.dtype, group: Optional[dist.ProcessGroup] = None, device=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > self.MAX_RANKS:
            raise ValueError(f"symmetric kernels support up to {self.MAX_RANKS} ranks")
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dtype, self.numel = dtype, numel
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=self.device)
        self._h_data = symm_mem.rendezvous(self.tensor, group)
        self.pad = symm_mem.empty(64, dtype=torch.int32, device=self.device)
        self.pad.zero_()
        self._h_pad = symm_mem.rendezvous(self.pad, group)
        self.counter = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.seq = 0                      # uses of this buffer by a collective kernel so far
        self._chan_seq = [0, 0, 0, 0]     # last value signalled per channel by signal()
        self._data_ptrs = (ctypes.c_ulonglong * self.world)(*[int(p) for p in self._h_data.buffer_ptrs])
        self._pad_ptrs = (ctypes.c_ulonglong * self.world)(*[int(p) for p in self._h_pad.buffer_ptrs])
        mc = int(getattr(self._h_data, "multicast_ptr", 0) or 0)
        self.multicast_ptr = mc
        self.use_nvls = bool(mc) and nvls_wanted()
        self._peer_views: Optional[List[torch.Tensor]] = None
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    # ------------------------------------------------------------------------------------------
    def _head(self):
        self.seq += 1
        return (self._data_ptrs, self._pad_ptrs, ctypes.c_ulonglong(self.multicast_ptr), _lib.ptr(self.counter),
                ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_uint(self.seq))

    def _tail(self, max_blocks, nvls=True):
        t = (ctypes.c_int(max_blocks), _lib.stream_ptr(), _lib.ptr(_lib.status_word(self.device)))
        return ((ctypes.c_int(int(self.use_nvls)),) + t) if nvls else t

    def check(self) -> None:
        """Synchronising check: raises if a cross-rank wait ran out."""
        try:
            _lib.check_status(self.device)
        except _lib.KernelError as e:
            raise CommTimeoutError(str(e)) from e

    def peer_view(self, rank: int) -> torch.Tensor:
        """Rank ``rank``'s copy of the buffer as a tensor on this device (peer memory)."""
        if self._peer_views is None:
            self._peer_views = [self._h_data.get_buffer(r, (self.numel,), self.dtype, 0) if r != self.rank
                                else self.tensor for r in range(self.world)]
        return self._peer_views[rank]

    # ----------------------------------------------------------------------------- flags
    def signal(self, channel: int, seq: Optional[int] = None) -> int:
        """On the current stream: tell every rank that this rank reached ``seq`` on ``channel``."""
        if seq is None:
            seq = self._chan_seq[channel] + 1
        self._chan_seq[channel] = seq
        rc = _lib.lib().atb_pad_signal(self._pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                       ctypes.c_uint(seq), ctypes.c_int(channel), _lib.stream_ptr())
        _lib.check(rc, "atb_pad_signal")
        return seq

    def wait(self, channel: int, seq: int) -> None:
        """On the current stream: wait (bounded) until every rank has signalled ``seq`` on ``channel``."""
        rc = _lib.lib().atb_pad_wait(self._pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                     ctypes.c_uint(seq), ctypes.c_int(channel), _lib.stream_ptr(),
                                     _lib.ptr(_lib.status_word(self.device)))
        _lib.check(rc, "atb_pad_wait")

    def wait_peers_done(self) -> None:
        """On the current stream: every rank has finished reading this buffer in its last collective
        kernel; the local copy may be overwritten afterwards."""
        if self.seq > 0:
            self.wait(CH_DONE, self.seq)

    def resync(self) -> None:
        """After a timeout (a rank missed a call): with every rank idle and on the host, agree on the
        highest sequence number and bring all channels of all pads up to it, so that the next call
        starts from a consistent state. Collective over the buffer's group."""
        torch.cuda.synchronize(self.device)
        t = torch.tensor([self.seq], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        self.seq = int(t.item())
        for ch in (CH_ARRIVE, CH_MID, CH_DONE):
            self.signal(ch, self.seq)
        self.counter.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------------- collectives
    def all_reduce_(self, scale: float = 1.0, numel: Optional[int] = None, max_blocks: int = 0,
                    offset: int = 0) -> torch.Tensor:
        """In-place all-reduce (sum * scale) of ``tensor[offset : offset + numel]``."""
        n = (self.numel - offset) if numel is None else numel
        rc = _lib.lib().atb_p2p_allreduce(*self._head(), ctypes.c_longlong(n), ctypes.c_longlong(offset),
                                          ctypes.c_float(scale),
                                          ctypes.c_int(_lib.DT[self.dtype]), *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_allreduce")
        return self.tensor

    def reduce_scatter_adamw(self, master, m, v, lp, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                             grad_out=None, numel: Optional[int] = None, max_blocks: int = 0) -> None:
        n = self.numel if numel is None else numel
        rc = _lib.lib().atb_p2p_rs_adamw(*self._head(), ctypes.c_longlong(n), _lib.ptr(master), _lib.ptr(m),
                                         _lib.ptr(v), _lib.ptr(lp), _lib.ptr(grad_out), ctypes.c_float(lr),
                                         ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
                                         ctypes.c_float(weight_decay), ctypes.c_int(step), ctypes.c_float(grad_scale),
                                         ctypes.c_int(_lib.DT[self.dtype]), *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_rs_adamw")

    def reduce_scatter_into(self, out: torch.Tensor, scale: float = 1.0, accumulate: bool = False,
                            numel: Optional[int] = None, max_blocks: int = 0) -> None:
        n = self.numel if numel is None else numel
        assert out.dtype == torch.float32
        rc = _lib.lib().atb_p2p_reduce_scatter(*self._head(), ctypes.c_longlong(n), _lib.ptr(out),
                                               ctypes.c_float(scale), ctypes.c_int(int(accumulate)),
                                               ctypes.c_int(_lib.DT[self.dtype]), *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_reduce_scatter")

    def allreduce_nesterov(self, synced, momentum_buf, lr, momentum, nesterov, first_step, clip_scale=1.0,
                           max_blocks: int = 0) -> None:
        assert self.dtype == torch.float32
        rc = _lib.lib().atb_p2p_allreduce_nesterov(*self._head(), ctypes.c_longlong(self.numel), _lib.ptr(synced),
                                                   _lib.ptr(momentum_buf), ctypes.c_float(lr),
                                                   ctypes.c_float(momentum), ctypes.c_int(int(nesterov)),
                                                   ctypes.c_int(int(first_step)), ctypes.c_float(clip_scale),
                                                   *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_allreduce_nesterov")

    def all_gather_into(self, out: torch.Tensor, max_blocks: int = 0) -> None:
        nbytes = self.numel * self.tensor.element_size()
        assert out.numel() * out.element_size() == nbytes * self.world
        self.seq += 1
        rc = _lib.lib().atb_p2p_allgather(self._data_ptrs, self._pad_ptrs, _lib.ptr(self.counter),
                                          ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_uint(self.seq),
                                          ctypes.c_longlong(nbytes), _lib.ptr(out),
                                          *self._tail(max_blocks, nvls=False))
        _lib.check(rc, "atb_p2p_allgather")

    def copy_engine_all_gather(self, out: torch.Tensor, offset: int = 0, numel: Optional[int] = None) -> None:
        """``out[p*n:(p+1)*n] = rank p's buffer[offset:offset+n]`` for every rank p, as one device-to-device
        copy per rank on the current stream, starting with the next rank so that no rank is read by
        everybody at once. The caller orders it after the peers' data is in place (``wait(CH_READY, ..)``)."""
        n = (self.numel - offset) if numel is None else numel
        assert out.numel() == n * self.world and out.dtype == self.dtype
        for k in range(self.world):
            p = (self.rank + 1 + k) % self.world
            out[p * n: (p + 1) * n].copy_(self.peer_view(p)[offset: offset + n], non_blocking=True)


# ----------------------------------------------------------------------------------------------
# all-to-all by pulls: every rank publishes ``send [W, chunk]`` in symmetric memory and copies, with the copy
# engines, chunk ``rank`` of every peer's buffer into ``recv [W, chunk]`` (what dist.all_to_all_single does, without
# a collective kernel on the SMs). Used by the Ulysses head <-> sequence exchange.
# ----------------------------------------------------------------------------------------------
_a2a_buffers: dict = {}


def all_to_all_available(x: torch.Tensor, group) -> bool:
    return (x.is_cuda and available() and 1 < dist.get_world_size(group) <= SymmetricBuffer.MAX_RANKS
            and (x.numel() * x.element_size()) % 16 == 0)


def all_to_all_pull(send: torch.Tensor, group) -> torch.Tensor:
    """``recv[p] = rank p's send[rank]`` for ``send`` of shape ``[W, ...]`` (contiguous)."""
    W, r = dist.get_world_size(group), dist.get_rank(group)
    assert send.shape[0] == W and send.is_contiguous()
    key = (id(group), send.numel(), send.dtype, send.device.index)
    buf = _a2a_buffers.get(key)
    if buf is None:
        buf = _a2a_buffers[key] = SymmetricBuffer(send.numel(), send.dtype, group, send.device)
    if buf.seq > 0:
        buf.wait(CH_DONE, buf.seq)                 # every peer has read the previous contents
    buf.tensor.copy_(send.reshape(-1))
    buf.seq += 1
    buf.signal(CH_READY, buf.seq)
    buf.wait(CH_READY, buf.seq)                    # every rank has published
    recv = torch.empty_like(send)
    n = send.numel() // W
    flat = recv.view(W, n)
    for k in range(W):
        p = (r + k) % W
        flat[p].copy_(buf.peer_view(p)[r * n: (r + 1) * n], non_blocking=True)
    buf.signal(CH_DONE, buf.seq)
    return recv
