"""Dry run of a candidate strategy: build it on a deep copy of the model context, run warm-up and
timed steps, report throughput (samples/s), data-loading share and peak memory. Out-of-memory or
any failure counts as throughput 0.
(Reference: atorch/auto/dry_runner/dry_runner.py:12-136; step counts from ATORCH_DRYRUN_WARMUP_STEP /
ATORCH_DRYRUN_PROFILE_STEP.)
"""
from __future__ import annotations

import copy
import logging
import os
import time
from typing import Optional

import torch

logger = logging.getLogger("atorch.logger")


def profile_context(mc, warmup: Optional[int] = None, steps: Optional[int] = None) -> dict:
    warmup = int(os.environ.get("ATORCH_DRYRUN_WARMUP_STEP", 10)) if warmup is None else warmup
    steps = int(os.environ.get("ATORCH_DRYRUN_PROFILE_STEP", 15)) if steps is None else steps
    if mc.dataloader is None and mc.sample_batch is None:
        mc.update_dataloader()
    it = iter(mc.dataloader) if mc.dataloader is not None else None
    cuda = torch.cuda.is_available()

    def next_batch():
        nonlocal it
        if it is None:
            return mc.sample_batch
        try:
            return next(it)
        except StopIteration:
            it = iter(mc.dataloader)
            return next(it)

    if cuda:
        torch.cuda.reset_peak_memory_stats()
    data_t = 0.0
    bs = None
    for i in range(warmup + steps):
        if i == warmup:
            if cuda:
                torch.cuda.synchronize()
            t0 = time.time()
            data_t = 0.0
        d0 = time.time()
        batch = next_batch()
        data_t += time.time() - d0
        if bs is None:
            first = batch[0] if isinstance(batch, (tuple, list)) else (next(iter(batch.values()))
                                                                         if isinstance(batch, dict) else batch)
            bs = first.shape[0] if hasattr(first, "shape") else 1
        mc.run_one_step(batch)
    if cuda:
        torch.cuda.synchronize()
    total = max(time.time() - t0, 1e-9)
    return {"throughput": steps * (bs or 1) / total, "data_loading_ratio": data_t / total,
            "max_gpu_memory": torch.cuda.max_memory_allocated() if cuda else 0, "step_time": total / steps}


def dry_run_strategy(mc, strategy, opt_lib, warmup: Optional[int] = None, steps: Optional[int] = None):
    from .accelerate import model_transform

    try:
        ctx = copy.deepcopy(mc)
        ctx = model_transform(ctx, copy.deepcopy(strategy), opt_lib)
        return profile_context(ctx, warmup, steps)
    except Exception as e:   # OOM and friends: the candidate is simply not viable
        logger.warning("dry run failed for %s: %s", strategy, e)
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        return {"throughput": 0.0, "error": str(e)}
