"""Long-context attention over a sequence-parallel group: ring attention (flash kernels per chunk, K/V chunks pulled
over peer memory) against Ulysses (head <-> sequence exchange around the flash kernels), forward + backward.

    torchrun --nproc-per-node N -m atorch_b200.benchmarks.ring_attn_bench [--seq-per-gpu 8192] [--heads 32] [--tiny]

Every rank holds ``seq-per-gpu`` tokens of q, k, v (``[1, S/N, H, 128]`` bf16, causal). Device-timed with CUDA events,
MAX over ranks; FLOPs counted for the whole causal sequence (4 S^2 H D / 2 forward, 2.5x that backward).
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from atorch_b200.benchmarks.common import report, setup, timed_steps
from atorch_b200.parallel.sequence_parallel import UlyssesAttention, ring_attention


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-per-gpu", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tiny", action="store_true")
    a = ap.parse_args(argv)
    rank, world, dev = setup()
    S_loc, H, D = (256, 4, 128) if a.tiny else (a.seq_per_gpu, a.heads, 128)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    g = torch.Generator().manual_seed(5 + rank)
    q, k, v = ((0.5 * torch.randn(1, S_loc, H, D, generator=g)).to(dev, dtype).requires_grad_() for _ in range(3))
    dy = torch.randn(1, S_loc, H, D, generator=g).to(dev, dtype)
    group = dist.group.WORLD if dist.is_initialized() else None
    ul = UlyssesAttention(causal=True)
    ul.set_sp(world, rank, group)

    def run(fn):
        def step(_):
            for t in (q, k, v):
                t.grad = None
            fn().backward(dy)
        return timed_steps(step, a.steps, a.warmup, dev) / a.steps

    S = S_loc * world
    flops = 3.5 * 4.0 * S * S * H * D * 0.5          # forward + backward, causal
    res = {}
    cases = [("ring", lambda: ring_attention(q, k, v, group, causal=True)), ("ulysses", lambda: ul(q, k, v))]
    if dev.type == "cuda" and world > 1:     # the same tensors read as the load-balanced layout (timing only)
        cases.insert(1, ("ring_zigzag", lambda: ring_attention(q, k, v, group, causal=True, layout="zigzag")))
    for name, fn in cases:
        if name == "ulysses" and H % world:
            continue
        ms = run(fn)
        res[name] = {"ms": round(ms, 3), "tflops_per_gpu": round(flops / world / ms / 1e9, 1)}
    report(rank, {"metric": "long-context attention fwd+bwd, sequence parallel", "n_gpus": world, "seq_len": S, "heads": H,
            "head_dim": D, "causal": True, "dtype": str(dtype).replace("torch.", ""), **res})


if __name__ == "__main__":
    main()
