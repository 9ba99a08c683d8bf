"""Dataloaders with relaxed ordering.

``UnorderedDataLoader`` yields batches in the order worker processes finish them (no head-of-line
blocking behind a slow sample); ``UnshuffledBatchDataLoader`` shuffles at batch granularity: samples
inside a batch stay consecutive (good for length-bucketed data), the batch order is permuted.
(Reference: atorch/data/unordered_dataloader.py, unshuffled_batch_dataloader.py.)
"""
from __future__ import annotations

import queue
import threading
from typing import Iterator, List

import torch
from torch.utils.data import DataLoader, Sampler


class UnorderedDataLoader:
    def __init__(self, dataset, batch_size: int = 1, num_workers: int = 2, collate_fn=None, drop_last: bool = False,
                 sampler=None, prefetch: int = 4):
        self.dataset, self.batch_size, self.num_workers = dataset, batch_size, max(num_workers, 1)
        self.collate_fn = collate_fn or torch.utils.data.default_collate
        self.drop_last, self.sampler, self.prefetch = drop_last, sampler, prefetch

    def _batches(self) -> List[List[int]]:
        idx = list(self.sampler) if self.sampler is not None else list(range(len(self.dataset)))
        out = [idx[i: i + self.batch_size] for i in range(0, len(idx), self.batch_size)]
        if self.drop_last and out and len(out[-1]) < self.batch_size:
            out.pop()
        return out

    def __len__(self):
        return len(self._batches())

    def __iter__(self):
        tasks: "queue.Queue" = queue.Queue()
        done: "queue.Queue" = queue.Queue(maxsize=self.prefetch * self.num_workers)
        batches = self._batches()
        for b in batches:
            tasks.put(b)

        def work():
            while True:
                try:
                    b = tasks.get_nowait()
                except queue.Empty:
                    return
                try:
                    done.put(self.collate_fn([self.dataset[i] for i in b]))
                except Exception as e:   # surface worker errors in the consumer
                    done.put(e)
        threads = [threading.Thread(target=work, daemon=True) for _ in range(self.num_workers)]
        for t in threads:
            t.start()
        for _ in range(len(batches)):
            item = done.get()
            if isinstance(item, Exception):
                raise item
            yield item


class _BatchShuffleSampler(Sampler):
    def __init__(self, n: int, batch_size: int, seed: int, rank: int = 0, num_replicas: int = 1):
        self.n, self.batch_size, self.seed, self.rank, self.num_replicas = n, batch_size, seed, rank, num_replicas
        self.epoch = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __iter__(self) -> Iterator[int]:
        nb = self.n // self.batch_size
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        order = torch.randperm(nb, generator=g).tolist()
        order = order[self.rank:: self.num_replicas]
        for b in order:
            yield from range(b * self.batch_size, (b + 1) * self.batch_size)

    def __len__(self):
        return (self.n // self.batch_size // self.num_replicas) * self.batch_size


class UnshuffledBatchDataLoader(DataLoader):
    def __init__(self, dataset, batch_size: int = 1, seed: int = 0, rank: int = 0, num_replicas: int = 1, **kw):
        kw.pop("shuffle", None)
        kw.pop("sampler", None)
        sampler = _BatchShuffleSampler(len(dataset), batch_size, seed, rank, num_replicas)
        super().__init__(dataset, batch_size=batch_size, sampler=sampler, **kw)

    def set_epoch(self, epoch: int) -> None:
        self.sampler.set_epoch(epoch)
