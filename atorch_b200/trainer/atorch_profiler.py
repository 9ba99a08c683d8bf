"""``get_profiler(args)``: the profiler object that ``ProfilerCallback`` drives.

* ``profiler_type=None`` or ``"nsys"``: a null context (an external tracer records; the callback only brackets
  the chosen steps);
* ``"nv"``: ``torch.profiler.profile`` with the wait / warmup / active / repeat / skip_first schedule of the
  arguments; ranks listed in ``profile_ranks`` (``[-1]`` = all) write a TensorBoard trace named
  ``torch_profiler_rank{r}_{host}_{pid}`` into ``profiler_file_path`` (gzipped when ``profile_use_gzip``),
  the others get a handler that writes nothing; ``profiler_config`` overrides any keyword;
* ``"nv_dp"``: the file-driven dynamic profiler (``utils/dynamic_profiler.py``) initialised from
  ``dynamic_profiler_config_path``;
* ``"hw"`` / ``"hw_dp"`` (Ascend profilers) do not exist on this hardware: a warning and a null context.

(Reference: atorch/trainer/atorch_profiler.py:13-160.)
"""
from __future__ import annotations

import os
import socket
from contextlib import nullcontext

from ..common.log_utils import default_logger as logger


def get_profiler(args):
    kind = getattr(args, "profiler_type", None)
    path = getattr(args, "profiler_file_path", None)
    if kind is None or kind == "nsys":
        return nullcontext()
    if kind == "nv":
        import torch

        if path is not None:
            os.makedirs(path, exist_ok=True)
        rank = getattr(args, "process_index", 0)
        ranks = getattr(args, "profile_ranks", [-1])
        if ranks == [-1] or rank in ranks:
            handler = torch.profiler.tensorboard_trace_handler(
                path or ".", worker_name=f"torch_profiler_rank{rank}_{socket.gethostname()}_{os.getpid()}",
                use_gzip=bool(getattr(args, "profile_use_gzip", False)))
        else:
            def handler(prof):          # this rank records but writes nothing
                return None
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        cfg = dict(activities=acts, with_stack=False, record_shapes=False, profile_memory=False,
                   schedule=torch.profiler.schedule(wait=args.profiler_schedule_wait,
                                                    warmup=args.profiler_schedule_warmup,
                                                    active=args.profiler_schedule_active,
                                                    repeat=getattr(args, "profiler_schedule_repeat", 1),
                                                    skip_first=getattr(args, "profiler_schedule_skip_first", 0)),
                   on_trace_ready=handler)
        cfg.update(getattr(args, "profiler_config", None) or {})
        return torch.profiler.profile(**cfg)
    if kind == "nv_dp":
        cfg_path = getattr(args, "dynamic_profiler_config_path", None)
        assert cfg_path is not None, "set 'dynamic_profiler_config_path' to use the dynamic profiler"
        try:
            from ..utils import dynamic_profiler

            dynamic_profiler.init(cfg_path)
        except Exception as e:  # noqa: BLE001 - profiling must never stop training
            logger.warning(f"dynamic profiler not started: {e}")
        return nullcontext()
    logger.warning(f"unsupported profiler_type {kind!r}; use one of 'nv', 'nv_dp', 'nsys'")
    return nullcontext()
