"""Shared-memory batch exchange between the ranks of one model-parallel group on a node.

One *writer* rank runs the real dataloader and publishes each batch into POSIX shared memory; the
*reader* ranks of the group (which must see identical data) attach and deserialize, so the dataset
is read and pre-processed once per group instead of once per rank. Slot protocol per group:
``shm_data_size`` slots, each with a header ``[seq, nbytes, n_read]``; the writer waits until all
readers consumed a slot (bounded by ``io_timeout``) before reusing it.
(Reference: atorch/data/shm_context.py:139-682, shm_dataloader.py:138-284.)
"""
from __future__ import annotations

import pickle
import struct
import time
from multiprocessing import shared_memory
from typing import Optional

_HDR = struct.Struct("<qqq")    # seq, nbytes, readers_done


class ShmDataContext:
    def __init__(self, is_master: bool, rank: int, group_size: int, shm_name_prefix: str = "atb_shm_",
                 shm_data_size: int = 2, slot_bytes: int = 64 << 20, io_timeout: float = 30.0,
                 initialize_timeout: float = 120.0):
        self.is_master, self.rank, self.readers = is_master, rank, group_size - 1
        self.nslots, self.slot_bytes, self.io_timeout = shm_data_size, slot_bytes, io_timeout
        self.name = f"{shm_name_prefix}data"
        total = self.nslots * (_HDR.size + slot_bytes)
        if is_master:
            try:
                old = shared_memory.SharedMemory(name=self.name)
                old.close()
                old.unlink()
            except FileNotFoundError:
                pass
            self.shm = shared_memory.SharedMemory(name=self.name, create=True, size=total)
            for s in range(self.nslots):
                _HDR.pack_into(self.shm.buf, self._off(s), -1, 0, self.readers)
        else:
            t0 = time.time()
            while True:
                try:
                    self.shm = shared_memory.SharedMemory(name=self.name)
                    break
                except FileNotFoundError:
                    if time.time() - t0 > initialize_timeout:
                        raise TimeoutError(f"shared memory {self.name} was not created in time")
                    time.sleep(0.05)
        self.seq = 0

    def _off(self, slot: int) -> int:
        return slot * (_HDR.size + self.slot_bytes)

    def _wait(self, cond, what: str):
        t0 = time.time()
        while not cond():
            if time.time() - t0 > self.io_timeout:
                raise TimeoutError(f"shm dataloader: timed out waiting for {what}")
            time.sleep(0.0005)

    def put(self, obj) -> None:
        payload = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        if len(payload) > self.slot_bytes:
            raise ValueError(f"batch of {len(payload)} bytes exceeds the slot size {self.slot_bytes}")
        off = self._off(self.seq % self.nslots)
        self._wait(lambda: _HDR.unpack_from(self.shm.buf, off)[2] >= self.readers, "readers to free a slot")
        self.shm.buf[off + _HDR.size: off + _HDR.size + len(payload)] = payload
        _HDR.pack_into(self.shm.buf, off, self.seq, len(payload), 0)
        self.seq += 1

    def get(self):
        off = self._off(self.seq % self.nslots)
        self._wait(lambda: _HDR.unpack_from(self.shm.buf, off)[0] == self.seq, "the writer")
        seq, n, done = _HDR.unpack_from(self.shm.buf, off)
        obj = pickle.loads(bytes(self.shm.buf[off + _HDR.size: off + _HDR.size + n]))
        # readers_done is incremented by each reader exactly once per slot use (single writer per field
        # would need one counter per reader; with few readers a compare-and-retry on the packed field suffices)
        _HDR.pack_into(self.shm.buf, off, seq, n, _HDR.unpack_from(self.shm.buf, off)[2] + 1)
        self.seq += 1
        return obj

    def close(self) -> None:
        self.shm.close()
        if self.is_master:
            try:
                self.shm.unlink()
            except FileNotFoundError:
                pass


class ShmDataloader:
    """Iterates batches: the writer rank pulls from ``DataLoader(dataset, **dataloader_args)`` and
    publishes, reader ranks receive. ``None`` marks the end of an epoch."""

    def __init__(self, dataset, dataloader_args: Optional[dict] = None, rank: int = 0, group_size: int = 1,
                 io_timeout: float = 30, initialize_timeout: float = 120, need_sync_write: bool = False,
                 shm_data_size: int = 2, shm_name_prefix: str = "atb_shm_", slot_bytes: int = 64 << 20):
        from torch.utils.data import DataLoader

        self.is_master = rank == 0
        self.ctx = ShmDataContext(self.is_master, rank, group_size, shm_name_prefix, shm_data_size, slot_bytes,
                                  io_timeout, initialize_timeout)
        self.loader = DataLoader(dataset, **(dataloader_args or {})) if self.is_master else None
        self.sampler = getattr(self.loader, "sampler", None)

    def set_epoch(self, epoch: int) -> None:
        if self.sampler is not None and hasattr(self.sampler, "set_epoch"):
            self.sampler.set_epoch(epoch)

    def __iter__(self):
        if self.is_master:
            for batch in self.loader:
                if self.ctx.readers > 0:
                    self.ctx.put(batch)
                yield batch
            if self.ctx.readers > 0:
                self.ctx.put(None)
        else:
            while True:
                batch = self.ctx.get()
                if batch is None:
                    return
                yield batch

    def close(self) -> None:
        self.ctx.close()


def build_shm_dataloader(dataset, sampler, args):
    """Used by ``ModelContext.create_dataloader``: ranks of one ``tensor``/``pipe`` group share batches."""
    from ..distributed import distributed as D

    group = "tensor" if D.parallel_group("tensor") is not None else None
    if group is None:
        return None
    _, ranks = D.parallel_group_and_ranks(group)
    a = dict(args)
    a["sampler"] = sampler
    return ShmDataloader(dataset, a, rank=D.parallel_rank(group), group_size=len(ranks),
                         shm_name_prefix=f"atb_shm_{ranks[0]}_")
