"""Symmetric (peer-mapped) buffers and the fused collective kernels that run on them.

``SymmetricBuffer(numel, dtype, group)`` allocates the same buffer on every rank of ``group`` with
``torch.distributed._symmetric_memory`` (CUDA VMM + handle exchange), so every rank holds device
addresses of all peers' copies, plus a small signal pad and a device-side sync record. The methods
launch the kernels of ``csrc/comm.cu``, which read the peers' data over NVLink from inside the
kernel that does the arithmetic:

* ``all_reduce_(scale)``                  two-shot all-reduce in place
* ``reduce_scatter_adamw(...)``           gradient reduce-scatter fused with the sharded AdamW step
* ``reduce_scatter_into(out, ...)``       reduce-scatter into a local fp32 shard (optionally accumulating)
* ``allreduce_nesterov(...)``             local-SGD outer step (pseudo-gradient mean + Nesterov + write-back)
* ``all_gather_into(out)``                pull every peer's buffer into a local tensor

All launches on one buffer must go to the same stream (their ordering is the protocol). A wait
that runs out raises ``CommTimeoutError`` at the next ``check()``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib


class CommTimeoutError(RuntimeError):
    pass


def available() -> bool:
    if not (torch.cuda.is_available() and dist.is_available() and dist.is_initialized()):
        return False
    L = _lib.lib()
    return L is not None and L.has("atb_p2p_allreduce")


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
        self.state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._data_ptrs = (ctypes.c_ulonglong * self.world)(*[int(p) for p in self._h_data.buffer_ptrs])
        self._pad_ptrs = (ctypes.c_ulonglong * self.world)(*[int(p) for p in self._h_pad.buffer_ptrs])
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    # ------------------------------------------------------------------------------------------
    def _common(self):
        return (self._data_ptrs, self._pad_ptrs, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                _lib.ptr(self.state))

    def _tail(self, max_blocks):
        return (ctypes.c_int(max_blocks), _lib.stream_ptr(), _lib.ptr(_lib.status_word(self.device)))

    def check(self) -> None:
        """Synchronising check: raises if a cross-rank wait ran out."""
        try:
            _lib.check_status(self.device)
        except _lib.KernelError as e:
            raise CommTimeoutError(str(e)) from e

    def all_reduce_(self, scale: float = 1.0, numel: Optional[int] = None, max_blocks: int = 0) -> torch.Tensor:
        n = self.numel if numel is None else numel
        rc = _lib.lib().atb_p2p_allreduce(*self._common(), ctypes.c_longlong(n), ctypes.c_float(scale),
                                          ctypes.c_int(_lib.DT[self.dtype]), *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_allreduce")
        return self.tensor

    def reduce_scatter_adamw(self, master, m, v, lp, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                             grad_out=None, numel: Optional[int] = None, max_blocks: int = 0) -> None:
        n = self.numel if numel is None else numel
        rc = _lib.lib().atb_p2p_rs_adamw(*self._common(), ctypes.c_longlong(n), _lib.ptr(master), _lib.ptr(m),
                                         _lib.ptr(v), _lib.ptr(lp), _lib.ptr(grad_out), ctypes.c_float(lr),
                                         ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
                                         ctypes.c_float(weight_decay), ctypes.c_int(step), ctypes.c_float(grad_scale),
                                         ctypes.c_int(_lib.DT[self.dtype]), *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_rs_adamw")

    def reduce_scatter_into(self, out: torch.Tensor, scale: float = 1.0, accumulate: bool = False,
                            numel: Optional[int] = None, max_blocks: int = 0) -> None:
        n = self.numel if numel is None else numel
        assert out.dtype == torch.float32
        rc = _lib.lib().atb_p2p_reduce_scatter(*self._common(), ctypes.c_longlong(n), _lib.ptr(out),
                                               ctypes.c_float(scale), ctypes.c_int(int(accumulate)),
                                               ctypes.c_int(_lib.DT[self.dtype]), *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_reduce_scatter")

    def allreduce_nesterov(self, synced, momentum_buf, lr, momentum, nesterov, first_step, clip_scale=1.0,
                           max_blocks: int = 0) -> None:
        assert self.dtype == torch.float32
        rc = _lib.lib().atb_p2p_allreduce_nesterov(*self._common(), ctypes.c_longlong(self.numel), _lib.ptr(synced),
                                                   _lib.ptr(momentum_buf), ctypes.c_float(lr),
                                                   ctypes.c_float(momentum), ctypes.c_int(int(nesterov)),
                                                   ctypes.c_int(int(first_step)), ctypes.c_float(clip_scale),
                                                   *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_allreduce_nesterov")

    def all_gather_into(self, out: torch.Tensor, max_blocks: int = 0) -> None:
        nbytes = self.numel * self.tensor.element_size()
        assert out.numel() * out.element_size() == nbytes * self.world
        rc = _lib.lib().atb_p2p_allgather(*self._common(), ctypes.c_longlong(nbytes), _lib.ptr(out),
                                          *self._tail(max_blocks))
        _lib.check(rc, "atb_p2p_allgather")
