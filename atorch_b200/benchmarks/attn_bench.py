"""Micro-benchmark of the sm_100a flash attention (forward, backward) against torch SDPA (cuDNN) and
flash_attn 2.8 (the kernel behind the reference's FlashAttnModule), when that package is importable.
The forward is timed for both kernels of this package (one query tile per CTA, two tiles per CTA), the
backward for both forms (key-block kernel + query-block kernel, or one key-block kernel with reduce-adds).

    python -m atorch_b200.benchmarks.attn_bench [--iters 10]
"""
from __future__ import annotations

import argparse
import math

import torch

from atorch_b200 import _lib
from atorch_b200.ops import flash


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
    return ts[len(ts) // 2] * 1e3


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    # the last two: head dim 64 (GPT-2 medium / BERT-large like); the others: head dim 128
    for (B, S, H, Hkv, causal, D) in [(1, 4096, 32, 32, True, 128), (1, 4096, 32, 32, False, 128),
                                      (4, 2048, 16, 16, True, 128), (1, 4096, 32, 8, True, 128),
                                      (1, 8192, 32, 32, True, 128), (8, 1024, 16, 16, True, 64),
                                      (16, 512, 16, 16, False, 64)]:
        q = torch.randn(B, S, H, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(B, S, Hkv, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn(B, S, Hkv, D, device=dev, dtype=torch.bfloat16, requires_grad=True)
        flops_f = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
        scale = 1.0 / math.sqrt(D)

        def ours_f():
            return flash.flash_fwd_raw(q, k, v, causal, scale, None, None)

        def lib_f():
            return torch.nn.functional.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal, enable_gqa=H != Hkv)
        flash.FWD_TWO_TILES = False
        t_o = time_fn(ours_f, args.iters, flush)
        flash.FWD_TWO_TILES = True
        t_o2 = time_fn(ours_f, args.iters, flush)
        flash.FWD_TWO_TILES = False
        t_l = time_fn(lib_f, args.iters, flush)
        _lib.check_status(dev)
        line = (f"B{B} S{S} H{H}/{Hkv} D{D} causal={int(causal)} fwd: ours {t_o:8.1f} us {flops_f / t_o / 1e6:7.1f} TF | "
                f"ours(2 tiles) {t_o2:8.1f} us {flops_f / t_o2 / 1e6:7.1f} TF | "
                f"SDPA {t_l:8.1f} us {flops_f / t_l / 1e6:7.1f} TF")
        fa = None
        try:
            from flash_attn import flash_attn_func as fa
        except Exception:
            pass
        if fa is not None:
            t_fa = time_fn(lambda: fa(q, k, v, causal=causal), args.iters, flush)
            line += f" | flash_attn {t_fa:8.1f} us {flops_f / t_fa / 1e6:7.1f} TF"
        if flash.backward_built():
            out, lse = ours_f()
            dout = torch.randn_like(out)

            def ours_b():
                return flash.flash_bwd_raw(dout, q, k, v, out, lse, causal, scale, None, None)
            o2 = lib_f()
            d2 = torch.randn_like(o2)

            def lib_b():
                return torch.autograd.grad(o2, (q, k, v), d2, retain_graph=True)
            saved = flash.BWD_SPLIT
            L = _lib.lib()
            flash.BWD_SPLIT = True
            L.atb_flash_bwd_set_dkv(-1)
            tb_o = time_fn(ours_b, args.iters, flush)            # default: dK/dV kernel chosen by shape + dQ kernel
            L.atb_flash_bwd_set_dkv(1)
            tb_o2 = time_fn(ours_b, args.iters, flush)           # transposed dK/dV kernel + dQ kernel
            L.atb_flash_bwd_set_dkv(-1)
            flash.BWD_SPLIT = False
            tb_o1 = time_fn(ours_b, args.iters, flush)           # one key-block kernel, dQ by TMA reduce-adds
            flash.BWD_SPLIT = saved
            tb_l = time_fn(lib_b, args.iters, flush)
            _lib.check_status(dev)
            line += (f" || bwd: ours {tb_o:8.1f} us {2.5 * flops_f / tb_o / 1e6:7.1f} TF | "
                     f"ours(transposed dK/dV) {tb_o2:8.1f} us | ours(one kernel) {tb_o1:8.1f} us | "
                     f"SDPA {tb_l:8.1f} us {2.5 * flops_f / tb_l / 1e6:7.1f} TF")
            if fa is not None:
                o3 = fa(q, k, v, causal=causal)
                d3 = torch.randn_like(o3)
                tb_fa = time_fn(lambda: torch.autograd.grad(o3, (q, k, v), d3, retain_graph=True), args.iters, flush)
                line += f" | flash_attn {tb_fa:8.1f} us {2.5 * flops_f / tb_fa / 1e6:7.1f} TF"
        print(line, flush=True)


if __name__ == "__main__":
    main()
