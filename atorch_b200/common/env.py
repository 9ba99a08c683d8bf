"""Typed settings with environment override (one object instead of scattered ``os.getenv`` calls).
(Reference: atorch/common/env.py:17-34 and the scattered ATORCH_* / MOE_* variables.)"""
from __future__ import annotations

import os


def _b(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    return default if v is None else v.lower() in ("1", "true", "yes", "on")


def _i(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


class EnvSetting:
    _inst = None

    def __new__(cls):
        if cls._inst is None:
            cls._inst = super().__new__(cls)
        cls._inst.refresh()
        return cls._inst

    def refresh(self) -> None:
        self.MOE_FSDP_PREFETCH_NUM = _i("MOE_FSDP_PREFETCH_NUM", 1)
        self.MOE_DISABLE_SHARED_EXPERT_OVERLAP = _b("MOE_DISABLE_SHARED_EXPERT_OVERLAP")
        self.ATORCH_DISABLE_CHECKPOINT_PATCH = _b("ATORCH_DISABLE_CHECKPOINT_PATCH")
        self.MOE_NV_DISABLE_FUSED_KERNEL = _b("MOE_NV_DISABLE_FUSED_KERNEL")
        self.MOE_MLP_PREFIX = _b("MOE_MLP_PREFIX")
        self.DISABLE_TE_LINEAR_PATCHING = _b("DISABLE_TE_LINEAR_PATCHING")
        self.DEBUG = _b("ATORCH_DEBUG")
        self.FORCE_FSDP2_RESHARD_AFTER_FORWARD = _b("FORCE_FSDP2_RESHARD_AFTER_FORWARD")
        self.CLOSE_FSDP2_BACKWARD_PREFETCH = _b("CLOSE_FSDP2_BACKWARD_PREFETCH")
        self.FORCE_QUANTIZE_PER_MICROBATCH = _b("FORCE_QUANTIZE_PER_MICROBATCH")
        self.ENABLE_SHM_DATALOADER = _b("ENABLE_SHM_DATALOADER")
        self.SHM_DATALOADER_IO_TIMEOUT = _i("SHM_DATALOADER_IO_TIMEOUT", 30)
        self.SHM_DATALOADER_INIT_TIMEOUT = _i("SHM_DATALOADER_INIT_TIMEOUT", 120)
        self.ATORCH_NCCL_EXEC_TIMEOUT = _i("ATORCH_NCCL_EXEC_TIMEOUT", 1800)
        self.ATORCH_DRYRUN_WARMUP_STEP = _i("ATORCH_DRYRUN_WARMUP_STEP", 10)
        self.ATORCH_DRYRUN_PROFILE_STEP = _i("ATORCH_DRYRUN_PROFILE_STEP", 15)
