"""Local SGD / EDiT benchmark: one model replica per GPU, inner AdamW, outer Nesterov every H steps.

    torchrun --nproc-per-node 8 -m atorch_b200.benchmarks.local_sgd_bench --H 32 [--tiny]
    ... --H 0    synchronous DDP baseline

Llama 1.3B (24 layers, hidden 2048, 16 heads, FFN 5504), seq 2048, micro-batch 4, inner AdamW lr 3e-4, outer
SGD lr 0.7 momentum 0.9 Nesterov. Times ``H`` inner steps plus one outer step per window.
"""
from __future__ import annotations

import argparse

import torch

from atorch_b200.auto import auto_accelerate
from atorch_b200.benchmarks.common import reference_unavailable, report, setup, timed_steps
from atorch_b200.local_sgd import (LocalSGDConfig, OuterOptimizerConfig, OuterOptimPeriodicModelAverager,
                                   StatefulPostLocalSGDOptimizer)
from atorch_b200.models.llama import LlamaConfig, LlamaDecoderLayer, LlamaModel


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--windows", type=int, default=2)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    a = ap.parse_args(argv)
    if a.impl == "reference":
        reference_unavailable("the reference's FSDP local-SGD patch rewrites torch 2.1 / 2.4 FSDP internals (atorch/local_sgd/FSDP/__init__.py) and has not been validated against the torch 2.11 of this image")
        return
    rank, world, dev = setup()
    cfg = LlamaConfig.tiny() if a.tiny else LlamaConfig.llama_1p3b()
    seq, mbs = (64, 2) if a.tiny else (2048, 4)
    torch.manual_seed(1234)
    with torch.device(dev):
        model = LlamaModel(cfg)
    if a.H == 0:          # synchronous data parallel
        strategy = ["parallel_mode", ("fsdp", {"atorch_wrap_cls": (LlamaDecoderLayer,)}),
                    ("amp_native", {"dtype": torch.bfloat16}), ("checkpoint", {"wrap_class": (LlamaDecoderLayer,)})]
    else:                 # every rank trains its own replica: the sharded engine at shard-group size 1
        strategy = [("fsdp", {"atorch_wrap_cls": (LlamaDecoderLayer,),
                              "process_group": torch.distributed.new_group([rank]) if world > 1 else None}),
                    ("amp_native", {"dtype": torch.bfloat16}), ("checkpoint", {"wrap_class": (LlamaDecoderLayer,)})]
        if world > 1:
            for r in range(world):      # new_group is collective: every rank creates every singleton group
                if r != rank:
                    torch.distributed.new_group([r])
    ok, res, _ = auto_accelerate(model, torch.optim.AdamW, loss_func=lambda b, o: o[0], optim_args={"lr": 3e-4},
                                 load_strategy=strategy)
    assert ok
    optim = res.optim
    if a.H > 0 and world > 1:
        eng = res.model.engine
        avg = OuterOptimPeriodicModelAverager(
            local_sgd_config=LocalSGDConfig(local_sgd_sync_interval=a.H, local_sgd_warmup_steps=0),
            outer_optim_config=OuterOptimizerConfig(torch.optim.SGD, {"lr": 0.7, "momentum": 0.9, "nesterov": True}))
        master = torch.nn.Parameter(eng.master)          # the whole replica is one flat fp32 tensor

        class _Opt:
            param_groups = [{"params": [master]}]

            def step(self_inner):
                optim.step()

            def zero_grad(self_inner, set_to_none=True):
                optim.zero_grad()

            def state_dict(self_inner):
                return {}
        lopt = StatefulPostLocalSGDOptimizer(_Opt(), avg)
        post_sync = eng.sync_working_copy
    else:
        lopt, avg, post_sync = optim, None, None
    ids = torch.randint(0, cfg.vocab_size, (mbs, seq), device=dev)

    def step(i):
        lopt.zero_grad()
        loss = res.model(input_ids=ids, labels=ids, return_logits=False)[0]
        loss.backward()
        lopt.step()
        if avg is not None and (avg.step - 1) % a.H == 0:
            post_sync()                                   # refresh the bf16 working copy after an outer step
        return loss
    steps = max(a.H, 1) * a.windows
    ms = timed_steps(step, steps, max(a.H, 1), dev)
    report(rank, {"metric": "tokens/sec local SGD (device-timed, max over ranks)",
                  "value": round(world * mbs * seq * steps / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
                  "ms_per_step": round(ms / steps, 2), "config": {"model": "tiny" if a.tiny else "llama-1.3b",
                  "H": a.H, "seq_len": seq, "micro_batch": mbs, "outer": "SGD lr 0.7 momentum 0.9 nesterov",
                  "mode": "sync fsdp" if a.H == 0 else "one replica per GPU"}})


if __name__ == "__main__":
    main()
