"""Runs one kernel a few times on a case sized for an ncu capture (inputs above the 126 MB L2, well
under a few GB): ``python -m atorch_b200.benchmarks.profile_case <case>`` with case one of
gemm | gemm1 | gemm_swiglu | gemm_grouped | flash_hd64 | flash_fwd | flash_bwd | rmsnorm | layernorm | rope | swiglu | ce | adamw | agd |
fp8_quant | fp8_gemm | quant | moe | reduce_scatter. The last two run the peer-memory kernels on a process
group of one rank (the "peers" are this GPU), which exercises the same code without a second GPU.
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
    elif case == "gemm_swiglu":          # gate|up projection with SwiGLU in the epilogue, Llama-2 7B shape
        from atorch_b200.ops.gemm import gemm_swiglu

        x = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(2 * 11008, 4096, device=dev, dtype=torch.bfloat16) * 0.02
        for i in range(n):
            gemm_swiglu(x, w, keep_gate_up=bool(i & 1))        # without / with the pre-activation output
    elif case == "flash_hd64":           # head dim 64: single-tile forward, one-kernel backward
        q, k, v = (torch.randn(8, 1024, 16, 64, device=dev, dtype=torch.bfloat16) for _ in range(3))
        for _ in range(n):
            out, lse = flash.flash_fwd_raw(q, k, v, True, 0.125, None, None)
            flash.flash_bwd_raw(torch.ones_like(out), q, k, v, out, lse, True, 0.125, None, None)
    elif case == "gemm_grouped":
        E, W, cap, K, N = 1, 8, 1280, 4096, 4096
        x = torch.randn(E * W * cap, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        counts = torch.tensor([1024, 900, 1280, 700, 1100, 1000, 1200, 990], dtype=torch.int32, device=dev)
        for _ in range(n):
            ops.gemm(x, w, groups={"counts": counts, "m_rows": cap})
    elif case == "layernorm":
        x = torch.randn(16384, 4096, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(4096, device=dev, dtype=torch.bfloat16, requires_grad=True)
        b = torch.zeros(4096, device=dev, dtype=torch.bfloat16, requires_grad=True)
        for _ in range(n):
            ops.layer_norm(x, w, b).backward(torch.ones_like(x))
    elif case == "rope":
        qkv = torch.randn(4, 4096, 96, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
        cos, sin = ops.rope_tables(4096, 128, 10000.0, dev)
        for _ in range(n):
            ops.rope(qkv.view(4, 4096, -1), cos, sin, 64, 128, inplace=True).backward(torch.ones(4, 4096, 96 * 128, device=dev,
                                                                                   dtype=torch.bfloat16))
    elif case == "swiglu":
        x = torch.randn(16384, 22016, device=dev, dtype=torch.bfloat16, requires_grad=True)
        for _ in range(n):
            ops.swiglu(x).backward(torch.ones(16384, 11008, device=dev, dtype=torch.bfloat16))
    elif case == "agd":
        m = 1 << 28
        master, a, b = (torch.zeros(m, device=dev) for _ in range(3))
        g = torch.randn(m, device=dev, dtype=torch.bfloat16)
        lp = torch.empty(m, device=dev, dtype=torch.bfloat16)
        for i in range(n):
            ops.agd_step(master, a, b, g, lp, 1e-3, 0.9, 0.999, 1e-5, 0.0, i + 1)
    elif case in ("fp8_quant", "fp8_gemm"):
        from atorch_b200.modules.fp8 import quantize as Q

        x = torch.randn(10240, 4096, device=dev, dtype=torch.bfloat16)
        w = (0.05 * torch.randn(8192, 4096, device=dev)).bfloat16()
        for _ in range(n):
            xq, xs = Q.tile_quantize(x)
            wq, ws, _ = Q.block_quantize(w, with_transpose=True)
            Q.tile_quantize_transposed(x)
        if case == "fp8_gemm":
            for _ in range(n):
                Q.scaled_gemm(xq, xs, wq, ws)
    elif case == "quant":
        from atorch_b200.ops.quantizer import CUDAQuantizer

        x = torch.randn(1 << 27, device=dev, dtype=torch.float16)
        qz = CUDAQuantizer(group_size=2048)
        for _ in range(n):
            q, p = qz.quantize(x, 8)
            qz.dequantize(q, p, 8)
    elif case in ("moe", "reduce_scatter"):
        import os

        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", torch.cuda.current_device()))
        if case == "reduce_scatter":
            from atorch_b200.parallel.symm import SymmetricBuffer

            buf = SymmetricBuffer(1 << 27, torch.bfloat16)
            buf.use_nvls = False
            buf.tensor.normal_()
            out = torch.empty(1 << 27, device=dev)
            m, v, master = (torch.zeros(1 << 27, device=dev) for _ in range(3))
            lp = torch.empty(1 << 27, device=dev, dtype=torch.bfloat16)
            for i in range(n):
                buf.reduce_scatter_into(out, scale=1.0, max_blocks=32)
                buf.reduce_scatter_adamw(master, m, v, lp, 1e-3, 0.9, 0.999, 1e-8, 0.01, i + 1, max_blocks=32)
            buf.check()
        else:
            from atorch_b200.modules.moe import peer_dispatch as pd

            T, k, E, H = 32768, 2, 8, 4096
            cap = pd.expert_capacity(T, k, E, 1.25)
            bufs = pd.PeerExpertBuffers(dist.group.WORLD, E, cap, H, dev)
            x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
            idx = torch.randint(0, E, (T, k), device=dev)
            w = torch.rand(T * k, device=dev)
            for _ in range(n):
                slot, count = pd.route(idx, E, cap)
                pd._scatter(bufs, bufs.X, x, idx, slot, None, count, k)
                rows = pd._take(bufs, bufs.X)
                pd._publish(bufs, bufs.Y, rows)
                pd._gather(bufs, bufs.Y, idx, slot, w, T, k)
        torch.cuda.synchronize()
        dist.destroy_process_group()
    else:
        raise SystemExit(f"unknown case {case}")
    torch.cuda.synchronize()
    _lib.check_status(dev)
    print(f"{case}: ok")


if __name__ == "__main__":
    main()
