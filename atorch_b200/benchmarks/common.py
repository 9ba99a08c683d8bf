"""Shared helpers of the benchmark scripts: rank setup, device-timed step loops (CUDA events, barrier and
synchronize on both sides, MAX over ranks), one JSON line on rank 0."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

import torch
import torch.distributed as dist


def setup():
    import atorch_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    if world > 1 or os.environ.get("ATB_FORCE_DIST"):
        atorch_b200.init_distributed("nccl" if cuda else "gloo", set_cuda_device_using_local_rank=cuda)
    rank = dist.get_rank() if dist.is_initialized() else 0
    return rank, world, torch.device("cuda", local) if cuda else torch.device("cpu")


def timed_steps(step: Callable[[int], object], steps: int, warmup: int, device) -> float:
    """Milliseconds for ``steps`` calls of ``step`` after ``warmup`` calls; MAX over ranks."""
    for i in range(warmup):
        step(i)
    cuda = device.type == "cuda"

    def fence():
        if dist.is_initialized():
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()
    fence()
    if cuda:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
    else:
        import time

        t0 = time.time()
    for i in range(steps):
        step(warmup + i)
    if cuda:
        e.record()
    fence()
    ms = s.elapsed_time(e) if cuda else (time.time() - t0) * 1e3
    t = torch.tensor([ms], device=device)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def report(rank: int, record: Dict) -> None:
    if rank == 0:
        print(json.dumps(record), flush=True)


def reference_unavailable(why: str) -> None:
    """The line a benchmark prints (rank 0) when its reference arm cannot run in this environment."""
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
