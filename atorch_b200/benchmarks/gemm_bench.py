"""Micro-benchmark of the tcgen05 bf16 GEMM against ``torch.matmul`` (cuBLAS) on the Llama shapes.

CUDA-event timing after warm-up, L2 flushed between iterations by writing a 256 MB buffer.
Prints one line per shape/layout: microseconds and TFLOP/s for both, and the ratio.

    python -m atorch_b200.benchmarks.gemm_bench [--iters 20] [--json out.json]
"""
from __future__ import annotations

import argparse
import json

import torch

from atorch_b200 import _lib
from atorch_b200.ops import gemm

SHAPES = [
    # (M, N, K, label)
    (4096, 12288, 4096, "7B qkv fwd"),
    (4096, 4096, 4096, "7B o_proj fwd"),
    (4096, 22016, 4096, "7B gate_up fwd"),
    (4096, 4096, 11008, "7B down fwd"),
    (4096, 32000, 4096, "7B lm_head fwd"),
    (8192, 8192, 8192, "square 8k"),
]


def time_fn(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        evs.append((s, e))
    torch.cuda.synchronize()
    ts = sorted(s.elapsed_time(e) for s, e in evs)
    return ts[len(ts) // 2] * 1e3  # median, microseconds


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", type=str, default=None)
    args = ap.parse_args(argv)
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for M, N, K, label in SHAPES:
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        cases = [
            ("fwd  x@W^T", lambda kn: gemm(x, w, kernel=kn), lambda: torch.matmul(x, w.t())),
            ("dgrad dy@W", lambda kn: gemm(dy, w, b_mn=True, kernel=kn), lambda: torch.matmul(dy, w)),
            ("wgrad dy^T@x", lambda kn: gemm(dy, x, a_mn=True, b_mn=True, kernel=kn), lambda: torch.matmul(dy.t(), x)),
        ]
        for name, ours_k, lib in cases:
            t_1 = time_fn(lambda: ours_k("1cta"), args.iters, flush)
            t_2 = time_fn(lambda: ours_k("2cta"), args.iters, flush)
            t_ours = min(t_1, t_2)
            t_lib = time_fn(lib, args.iters, flush)
            _lib.check_status(dev)
            row = dict(shape=label, M=M, N=N, K=K, op=name, ours_us=round(t_ours, 1), cta1_us=round(t_1, 1),
                       cta2_us=round(t_2, 1), cublas_us=round(t_lib, 1),
                       ours_tflops=round(flops / t_ours / 1e6, 1), cublas_tflops=round(flops / t_lib / 1e6, 1),
                       ratio=round(t_lib / t_ours, 3))
            rows.append(row)
            print(f"{label:16s} {name:14s} 1cta {t_1:8.1f} 2cta {t_2:8.1f} us best {row['ours_tflops']:7.1f} TF | "
                  f"cuBLAS {t_lib:8.1f} us {row['cublas_tflops']:7.1f} TF | ratio {row['ratio']:.3f}", flush=True)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
