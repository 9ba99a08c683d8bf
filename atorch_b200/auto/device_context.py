"""Facts about the machine the job runs on, used by planners and the dry run.

Numbers are those of an 8 x B200 NVSwitch node (per GPU: 180 GB HBM3e, NVLink 5 at 900 GB/s per
direction to every peer); the reference hard-codes A100 values in atorch/auto/device_context.py:41-52.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch

from ..distributed import distributed as D


class DeviceContext:
    def __init__(self):
        self.refresh()

    def refresh(self):
        self.node_num = D.node_size() or 1
        self.nproc_per_node = D.nproc_per_node() or 1
        self.cpu_num_per_node = os.cpu_count() or 1
        self.gpu_num_per_node = torch.cuda.device_count() if torch.cuda.is_available() else 0
        if torch.cuda.is_available():
            prop = torch.cuda.get_device_properties(torch.cuda.current_device())
            self.gpu_memory = prop.total_memory
            self.gpu_compute_capability = f"{prop.major}.{prop.minor}"
            self.sm_count = prop.multi_processor_count
        else:
            self.gpu_memory, self.gpu_compute_capability, self.sm_count = 0, None, 0
        peaks = self._measured_peaks()
        self.intra_node_bandwidth = 770e9      # measured peer copy, bytes/s per direction
        self.inter_node_bandwidth = 50e9
        self.hbm_bandwidth = peaks.get("hbm_gbs", 6650.0) * 1e9
        self.bf16_flops = peaks.get("bf16_tflops_sustained", 1400.0) * 1e12
        self.fp32_flops = 75e12

    @staticmethod
    def _measured_peaks() -> dict:
        p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
        try:
            return json.loads(p.read_text())
        except Exception:
            return {}

    @property
    def total_process(self) -> int:
        return self.node_num * self.nproc_per_node

    @property
    def context(self) -> dict:
        return dict(vars(self))


_ctx = None


def get_device_context() -> DeviceContext:
    global _ctx
    if _ctx is None:
        _ctx = DeviceContext()
    else:
        _ctx.refresh()
    return _ctx
