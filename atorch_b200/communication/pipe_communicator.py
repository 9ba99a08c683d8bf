"""Point-to-point transport of pipeline stages over NCCL (or gloo) send/recv.

The receiver does not know shapes in advance, so the first message of a given ``meta_id`` is
preceded by a two-step handshake of int64 tensors: ``[tensor_num, total_ndim]`` and then, per
tensor, ``[ndim, dtype_id, requires_grad]`` followed by all shapes. The result is cached by
``meta_id``; later messages with the same id go straight to the payload. Receive buffers are cached
per (meta_id, slot) and payloads of one message are posted together with ``batch_isend_irecv``.
(Reference: atorch/communication/pipe_communicator.py:27-496.)
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32, torch.int16,
           torch.int8, torch.uint8, torch.bool]
_DTYPE_ID = {d: i for i, d in enumerate(_DTYPES)}


class RecvBuffer:
    """Cache of receive buffers keyed by (meta_id, slot): a steady-state schedule allocates nothing."""

    def __init__(self):
        self._bufs: Dict[Tuple, List[torch.Tensor]] = {}

    def get(self, key, metas, device) -> List[torch.Tensor]:
        b = self._bufs.get(key)
        if b is None:
            b = [torch.empty(shape, dtype=dtype, device=device) for shape, dtype, _ in metas]
            self._bufs[key] = b
        return b

    def clear(self):
        self._bufs.clear()


class PipeCommunicator:
    def __init__(self, group: Optional[dist.ProcessGroup] = None, device=None):
        self.group = group
        self.device = device if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and
            dist.get_backend(group) == "nccl" else torch.device("cpu"))
        self._sent_meta: set = set()
        self._recv_meta: Dict = {}
        self.buffers = RecvBuffer()

    # ------------------------------------------------------------------------------ handshake
    def _send_meta(self, tensors: Sequence[torch.Tensor], dst: int) -> None:
        head = torch.tensor([len(tensors), sum(t.dim() for t in tensors)], dtype=torch.int64, device=self.device)
        dist.send(head, dst, group=self.group)
        body = []
        for t in tensors:
            body += [t.dim(), _DTYPE_ID[t.dtype], int(t.requires_grad)]
        for t in tensors:
            body += list(t.shape)
        dist.send(torch.tensor(body, dtype=torch.int64, device=self.device), dst, group=self.group)

    def _recv_meta_from(self, src: int):
        head = torch.empty(2, dtype=torch.int64, device=self.device)
        dist.recv(head, src, group=self.group)
        n, total_ndim = (int(x) for x in head.tolist())
        body = torch.empty(3 * n + total_ndim, dtype=torch.int64, device=self.device)
        dist.recv(body, src, group=self.group)
        body = body.tolist()
        metas, off = [], 3 * n
        for i in range(n):
            nd, dt, rg = body[3 * i: 3 * i + 3]
            metas.append((tuple(body[off: off + nd]), _DTYPES[dt], bool(rg)))
            off += nd
        return metas

    # --------------------------------------------------------------------------------- payload
    def send(self, tensors: Sequence[torch.Tensor], dst: int, meta_id=None) -> List:
        tensors = [t.contiguous() for t in tensors]
        key = (meta_id, dst)
        if meta_id is None or key not in self._sent_meta:
            self._send_meta(tensors, dst)
            if meta_id is not None:
                self._sent_meta.add(key)
        ops = [dist.P2POp(dist.isend, t, dst, self.group) for t in tensors]
        return dist.batch_isend_irecv(ops) if ops else []

    def recv(self, src: int, meta_id=None, slot: int = 0) -> Tuple[List[torch.Tensor], List]:
        key = (meta_id, src)
        metas = self._recv_meta.get(key) if meta_id is not None else None
        if metas is None:
            metas = self._recv_meta_from(src)
            if meta_id is not None:
                self._recv_meta[key] = metas
        bufs = self.buffers.get((meta_id, src, slot), metas, self.device) if meta_id is not None else \
            [torch.empty(s, dtype=d, device=self.device) for s, d, _ in metas]
        ops = [dist.P2POp(dist.irecv, b, src, self.group) for b in bufs]
        works = dist.batch_isend_irecv(ops) if ops else []
        for b, (_, _, rg) in zip(bufs, metas):
            b.requires_grad_(False)
        return bufs, works

    def recv_wait(self, src: int, meta_id=None, slot: int = 0) -> List[torch.Tensor]:
        bufs, works = self.recv(src, meta_id, slot)
        for w in works:
            w.wait()
        return bufs

    def metas(self, src: int, meta_id):
        return self._recv_meta.get((meta_id, src))
