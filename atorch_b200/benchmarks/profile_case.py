"""Runs one kernel a few times on a case sized for an ncu capture (inputs above the 126 MB L2, well
under a few GB): ``python -m atorch_b200.benchmarks.profile_case gemm|gemm1|flash_fwd|flash_bwd|rmsnorm|ce|adamw``.
"""
from __future__ import annotations

import math
import sys

import torch

from atorch_b200 import _lib, ops
from atorch_b200.ops import flash


def main(argv=None):
    case = (argv or sys.argv[1:] or ["gemm"])[0]
    dev = torch.device("cuda")
    torch.manual_seed(0)
    n = 3
    if case in ("gemm", "gemm1"):
        x = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(11008, 4096, device=dev, dtype=torch.bfloat16)
        for _ in range(n):
            ops.gemm(x, w, kernel="2cta" if case == "gemm" else "1cta")
    elif case in ("flash_fwd", "flash_bwd"):
        q, k, v = (torch.randn(1, 4096, 32, 128, device=dev, dtype=torch.bfloat16) for _ in range(3))
        sc = 1 / math.sqrt(128)
        for _ in range(n):
            out, lse = flash.flash_fwd_raw(q, k, v, True, sc, None, None)
        if case == "flash_bwd":
            dout = torch.randn_like(out)
            for _ in range(n):
                flash.flash_bwd_raw(dout, q, k, v, out, lse, True, sc, None, None)
    elif case == "rmsnorm":
        x = torch.randn(16384, 4096, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(4096, device=dev, dtype=torch.bfloat16, requires_grad=True)
        for _ in range(n):
            ops.rms_norm(x, w).backward(torch.ones_like(x))
    elif case == "ce":
        logits = torch.randn(4096, 32000, device=dev, dtype=torch.bfloat16, requires_grad=True)
        labels = torch.randint(0, 32000, (4096,), device=dev)
        for _ in range(n):
            ops.cross_entropy(logits, labels).sum().backward()
    elif case == "adamw":
        m = 1 << 28
        master, a, b = (torch.zeros(m, device=dev) for _ in range(3))
        g = torch.randn(m, device=dev, dtype=torch.bfloat16)
        lp = torch.empty(m, device=dev, dtype=torch.bfloat16)
        for i in range(n):
            ops.adamw_step(master, a, b, g, lp, 1e-3, 0.9, 0.999, 1e-8, 0.01, i + 1)
    else:
        raise SystemExit(f"unknown case {case}")
    torch.cuda.synchronize()
    _lib.check_status(dev)
    print(f"{case}: ok")


if __name__ == "__main__":
    main()
