"""Elastic data sharding: workers pull index ranges ("shards") from a shard service, so the set of
workers may change during an epoch without losing or repeating samples.

``ShardService`` is the in-process implementation of the service (a thread-safe queue of
``[start, end)`` ranges with re-queueing of shards whose worker died); ``ElasticDataset`` turns it into
a map-style dataset view, ``get_elastic_dataloader`` wraps it.
(Reference: atorch/data/elastic_dataset.py:19-139, elastic_dataloader.py:20-331, which talk to the
external elasticai_api shard service.)
"""
from __future__ import annotations

import threading
from collections import deque
from typing import Callable, Dict, Optional, Tuple

from torch.utils.data import DataLoader, IterableDataset


class ShardService:
    def __init__(self, dataset_size: int, shard_size: int, num_epochs: int = 1, shuffle: bool = False, seed: int = 0):
        self.lock = threading.Lock()
        self.todo: deque = deque()
        self.doing: Dict[int, Tuple[int, int, int]] = {}
        self._next_id = 0
        import random

        rng = random.Random(seed)
        for e in range(num_epochs):
            shards = [(s, min(s + shard_size, dataset_size)) for s in range(0, dataset_size, shard_size)]
            if shuffle:
                rng.shuffle(shards)
            self.todo.extend(shards)

    def fetch(self, worker: int) -> Optional[Tuple[int, int, int]]:
        with self.lock:
            if not self.todo:
                return None
            s, e = self.todo.popleft()
            tid = self._next_id
            self._next_id += 1
            self.doing[tid] = (worker, s, e)
            return tid, s, e

    def report_done(self, task_id: int) -> None:
        with self.lock:
            self.doing.pop(task_id, None)

    def recover_worker(self, worker: int) -> int:
        """Re-queue the unfinished shards of a worker that left; returns how many."""
        with self.lock:
            lost = [(tid, v) for tid, v in self.doing.items() if v[0] == worker]
            for tid, (_, s, e) in lost:
                del self.doing[tid]
                self.todo.appendleft((s, e))
            return len(lost)

    def finished(self) -> bool:
        with self.lock:
            return not self.todo and not self.doing


class ElasticDataset(IterableDataset):
    def __init__(self, read_sample: Callable[[int], object], service: ShardService, worker: int = 0):
        self.read_sample, self.service, self.worker = read_sample, service, worker

    def __iter__(self):
        while True:
            task = self.service.fetch(self.worker)
            if task is None:
                return
            tid, s, e = task
            for i in range(s, e):
                yield self.read_sample(i)
            self.service.report_done(tid)


def get_elastic_dataloader(read_sample, dataset_size: int, batch_size: int, shard_size: Optional[int] = None,
                           num_epochs: int = 1, shuffle: bool = False, worker: int = 0, service=None, **kw):
    service = service or ShardService(dataset_size, shard_size or batch_size * 8, num_epochs, shuffle)
    return DataLoader(ElasticDataset(read_sample, service, worker), batch_size=batch_size, **kw)
