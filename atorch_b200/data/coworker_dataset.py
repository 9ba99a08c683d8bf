"""``CoworkerDataset`` / ``build_coworker_dataloader``: offload part of the sample preprocessing to coworkers
(CPU-only helper processes, reachable over gRPC).

The dataset yields indices; the work happens in ``collate_fn`` inside the dataloader workers. Two modes
(mutually exclusive, the first wins):

* ``num_rpc_workers > 0``: that many dataloader workers send *all* their samples to coworkers, the other
  ``num_workers - num_rpc_workers`` process locally;
* ``coworker_process_percentage > 0``: every worker sends that fraction of each batch to coworkers and
  processes the rest locally while the remote part is in flight.

Remote samples go out ``num_rpc_fuse`` at a time, round-robin over the worker's coworkers, all calls issued
before the first result is awaited. ``pre_process_fn`` always runs locally, ``process_fn`` where the sample
is processed. A sample whose processing returns None is replaced by a randomly drawn other sample when
``need_padding_for_none``. Coworker addresses come from ``coworker_addrs`` or the ``COWORKER_ADDRS``
environment variable (comma separated ``host:port``); training rank r uses the coworkers with
``index % num_trainers == r`` (or the single coworker ``r % num_coworkers`` when there are fewer coworkers
than trainers), and they are dealt out to the dataloader workers that use RPC in the same modular way.
Without coworkers everything runs locally.

(Reference: atorch/data/coworker_dataset.py:13-394; remote execution there is torch RPC, here the
``process`` method of ``service/coworker_data_service.py``.)"""
from __future__ import annotations

import os
import random
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, List, Optional, Sequence

import torch
from torch.utils.data import DataLoader, Dataset
from torch.utils.data.dataloader import default_collate

from ..common.log_utils import default_logger as logger


def _split_coworkers(addrs: Sequence[str], rank: int, num_trainers: int) -> List[str]:
    if not addrs:
        return []
    if len(addrs) < num_trainers:
        return [addrs[rank % len(addrs)]]
    return [a for i, a in enumerate(addrs) if i % num_trainers == rank]


class CoworkerDataset(Dataset):
    def __init__(self, process_fn: Callable, dataset_size: int, pre_process_fn: Optional[Callable] = None,
                 num_workers: int = 0, num_rpc_workers: int = 0, coworker_process_percentage: float = 0.0,
                 custom_collate_fn: Optional[Callable] = None, num_rpc_fuse: int = 4,
                 need_padding_for_none: bool = False, coworker_addrs: Optional[Sequence[str]] = None,
                 rank: Optional[int] = None, num_trainers: Optional[int] = None):
        self.process_fn, self.pre_process_fn, self.dataset_size = process_fn, pre_process_fn, dataset_size
        self.num_workers, self.num_rpc_workers = num_workers, num_rpc_workers
        self.coworker_process_percentage = coworker_process_percentage
        self.custom_collate_fn, self.num_rpc_fuse = custom_collate_fn, max(int(num_rpc_fuse), 1)
        self.need_padding_for_none = need_padding_for_none
        if coworker_addrs is None:
            env = os.environ.get("COWORKER_ADDRS", "")
            coworker_addrs = [a for a in env.split(",") if a]
        rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        num_trainers = int(os.environ.get("WORLD_SIZE", "1")) if num_trainers is None else num_trainers
        self.coworkers = _split_coworkers(list(coworker_addrs), rank, max(num_trainers, 1))
        self.num_coworkers = len(self.coworkers)
        if self.num_coworkers == 0:
            if num_rpc_workers or coworker_process_percentage:
                logger.warning("no coworkers found: all samples are preprocessed locally")
            self.num_rpc_workers, self.coworker_process_percentage = 0, 0.0
        if self.num_rpc_workers > self.num_workers > 0:
            logger.error(f"num_workers ({self.num_workers}) is smaller than num_rpc_workers ({self.num_rpc_workers})")
            self.num_rpc_workers = self.num_workers
        self.num_local_workers = max(self.num_workers - self.num_rpc_workers, 0) if self.num_rpc_workers else \
            self.num_workers
        self.num_workers_needs_rpc = self.num_rpc_workers if self.num_rpc_workers > 0 else \
            (max(self.num_workers, 1) if self.coworker_process_percentage > 0 else 0)
        self.coworkers_distribution = self._deal_coworkers()
        self._clients = None           # created lazily inside each dataloader worker process

    def _deal_coworkers(self) -> List[List[str]]:
        n = self.num_workers_needs_rpc
        if n == 0 or self.num_coworkers == 0:
            return []
        dist: List[List[str]] = [[] for _ in range(n)]
        if self.num_coworkers < n:
            for i in range(n):
                dist[i].append(self.coworkers[i % self.num_coworkers])
        else:
            for i, c in enumerate(self.coworkers):
                dist[i % n].append(c)
        return dist

    def __getitem__(self, index):
        return index

    def __len__(self):
        return self.dataset_size

    def get_collate_fn(self):
        return self.custom_collate_fn if self.custom_collate_fn is not None else default_collate

    # ---------------------------------------------------------------- processing
    def _local(self, item):
        x = self.pre_process_fn(item) if self.pre_process_fn is not None else item
        return self.process_fn(x)

    def _remote(self, items: list, slot: int) -> list:
        from ..service.rpc_clients import CoworkerRpcClient

        if self._clients is None:
            self._clients = {}
        addrs = self.coworkers_distribution[slot % len(self.coworkers_distribution)]
        pool = ThreadPoolExecutor(max_workers=max(len(addrs), 1))
        futs = []
        for k, i in enumerate(range(0, len(items), self.num_rpc_fuse)):
            chunk = items[i: i + self.num_rpc_fuse]
            if self.pre_process_fn is not None:
                chunk = [self.pre_process_fn(c) for c in chunk]
            addr = addrs[k % len(addrs)]
            cl = self._clients.get(addr)
            if cl is None:
                cl = self._clients[addr] = CoworkerRpcClient(addr)
            futs.append(pool.submit(cl.process, self.process_fn, chunk))
        out = []
        for f in futs:
            out.extend(f.result())
        pool.shutdown(wait=False)
        return out

    def collate_fn(self, batch):
        info = torch.utils.data.get_worker_info()
        worker_id = info.id if info is not None else 0
        n = len(batch)
        if self.num_workers_needs_rpc == 0:
            local = n
        elif self.num_rpc_workers > 0:
            local = n if worker_id < self.num_local_workers else 0
        else:
            local = n - int(self.coworker_process_percentage * n)
        remote = n - local
        results: list = []
        fut = pool = None
        if remote > 0:
            pool = ThreadPoolExecutor(max_workers=1)
            fut = pool.submit(self._remote, [batch[i] for i in range(remote)], worker_id)
        local_results = [self._local(batch[i]) for i in range(remote, n)]
        if fut is not None:
            results.extend(fut.result())
            pool.shutdown(wait=False)
        results.extend(local_results)
        if self.need_padding_for_none:
            for i, r in enumerate(results):
                tries = 0
                while r is None and tries < 1000:
                    r = self._local(random.randint(0, self.dataset_size - 1))
                    tries += 1
                results[i] = r
        return self.get_collate_fn()(results)


def build_coworker_dataloader(process_fn, dataset_size, pre_process_fn=None, num_workers=0, num_rpc_workers=0,
                              coworker_process_percentage=0, batch_size=1, shuffle=True, custom_collate_fn=None,
                              num_rpc_fuse=4, need_padding_for_none=False, coworker_addrs=None, **kwargs):
    if num_rpc_workers > 0 and coworker_process_percentage > 0:
        logger.warning("num_rpc_workers and coworker_process_percentage are both set: the percentage is ignored")
        coworker_process_percentage = 0
    ds = CoworkerDataset(process_fn, dataset_size, pre_process_fn, num_workers, num_rpc_workers,
                         coworker_process_percentage, custom_collate_fn, num_rpc_fuse, need_padding_for_none,
                         coworker_addrs)
    sampler = None
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        sampler = torch.utils.data.DistributedSampler(ds, shuffle=shuffle)
    return DataLoader(ds, batch_size=batch_size, shuffle=(shuffle and sampler is None), sampler=sampler,
                      num_workers=num_workers, collate_fn=ds.collate_fn, **kwargs)
