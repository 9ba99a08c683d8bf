"""Micro-benchmark of the block-scaled fp8 path on the expert shapes of the Mixtral-style benchmark:
the tcgen05 ``kind::f8f6f4`` GEMM with 1x128 activation scales and 128x128 weight scales
(csrc/fp8.cu) against this package's bf16 GEMM and against ``torch._scaled_mm`` (cuBLASLt, per-tensor
scales: the nearest library form), plus the quantiser kernels as achieved GB/s.

CUDA-event timing after warm-up, L2 flushed between iterations by writing a 256 MB buffer.

    python -m atorch_b200.benchmarks.fp8_bench [--iters 10]
"""
from __future__ import annotations

import argparse
import json

import torch

from atorch_b200 import ops
from atorch_b200.benchmarks.gemm_bench import time_fn
from atorch_b200.modules.fp8 import quantize as Q

SHAPES = [
    (10240, 28672, 4096, "expert gate|up  (EP8: 8 x 1280 slots)"),
    (10240, 4096, 14336, "expert down"),
    (4096, 4096, 4096, "dense 4k"),
]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for M, N, K, label in SHAPES:
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = (0.05 * torch.randn(N, K, device=dev)).bfloat16()
        flops = 2.0 * M * N * K
        xq, xs = Q.tile_quantize(x)
        wq, ws, _ = Q.block_quantize(w, with_transpose=True)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        t_fp8 = time_fn(lambda: Q.scaled_gemm(xq, xs, wq, ws, out=out), a.iters, flush)
        t_bf16 = time_fn(lambda: ops.gemm(x, w, out=out), a.iters, flush)
        rec = {"shape": [M, N, K], "label": label, "fp8_block_scaled_us": round(t_fp8, 1),
               "fp8_tflops": round(flops / t_fp8 / 1e6, 1), "bf16_us": round(t_bf16, 1),
               "bf16_tflops": round(flops / t_bf16 / 1e6, 1)}
        try:
            xe = x.to(torch.float8_e4m3fn)
            we = w.to(torch.float8_e4m3fn)
            one = torch.ones((), device=dev)
            t_lib = time_fn(lambda: torch._scaled_mm(xe, we.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16),
                            a.iters, flush)
            rec.update(scaled_mm_tensorwise_us=round(t_lib, 1), scaled_mm_tflops=round(flops / t_lib / 1e6, 1))
        except Exception as e:   # library form not available for this shape / build
            rec["scaled_mm"] = f"unavailable: {type(e).__name__}"
        t_q = time_fn(lambda: Q.tile_quantize(x), a.iters, flush)
        t_b = time_fn(lambda: Q.block_quantize(w, with_transpose=True), a.iters, flush)
        rec.update(tile_quant_us=round(t_q, 1), tile_quant_gbs=round(M * K * 3 / t_q / 1e3, 1),
                   block_quant_t_us=round(t_b, 1), block_quant_gbs=round(N * K * 4 / t_b / 1e3, 1))
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
