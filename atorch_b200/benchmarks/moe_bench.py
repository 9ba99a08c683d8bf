"""Mixtral-style MoE training step with expert parallelism and block-scaled fp8 expert GEMMs.

    torchrun --nproc-per-node 8 -m atorch_b200.benchmarks.moe_bench [--fp8 0|1] [--tiny]

Layout: every rank holds ``num_experts / world`` experts (expert parallel over all ranks, tokens exchanged
with all-to-all); attention / router / embeddings are sharded data parallel over all ranks. Expert weights
live outside the sharded engine (they are not replicas of each other) in bf16 with fp32 masters.
16 layers, hidden 4096, 32 q / 8 kv heads, 8 experts top-2, expert FFN 14336, seq 4096, micro-batch 1.
"""
from __future__ import annotations

import argparse

import torch

from atorch_b200.auto import auto_accelerate
from atorch_b200.benchmarks.common import reference_unavailable, report, setup, timed_steps
from atorch_b200.distributed import distributed as D
from atorch_b200.models.mixtral import MixtralConfig, MixtralDecoderLayer, MixtralModel
from atorch_b200.modules.moe import Grouped_GEMM_MoE
from atorch_b200.optimizers import BF16Optimizer


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--fp8", type=int, default=1)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--dispatcher", default="auto", choices=["auto", "PeerMemory", "AllToAll", "AllGather"],
                    help="auto: PeerMemory (capacity factor 1.25, own kernels over NVLink) on GPUs, AllToAll elsewhere")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    a = ap.parse_args(argv)
    if a.impl == "reference":
        reference_unavailable("the reference's FP8 grouped linear imports the `kitchen` package and its bf16 Grouped_GEMM_MoE imports `grouped_gemm`; neither is installed and no index is reachable")
        return
    rank, world, dev = setup()
    if world > 1:
        D.create_parallel_group(([("expert", world)], None))
    disp = a.dispatcher
    if disp == "auto":
        disp = "PeerMemory" if (dev.type == "cuda" and world > 1) else "AllToAll"
    kw = dict(use_expert_parallelism=world > 1, fp8_experts=bool(a.fp8), gradient_checkpointing=True,
              token_dispatcher_type=disp)
    if a.layers:
        kw["num_hidden_layers"] = a.layers
    cfg = MixtralConfig.tiny_moe(**kw) if a.tiny else MixtralConfig.mixtral_bench(**kw)
    seq = 64 if a.tiny else 4096
    torch.manual_seed(1234 + rank)                       # experts differ per rank; shared parts are synchronised below
    with torch.device(dev):                              # initialise directly on the device
        model = MixtralModel(cfg)
    expert_params = [p for m in model.modules() if isinstance(m, Grouped_GEMM_MoE) for p in m.parameters()]
    for p in expert_params:
        p.data = p.data.to(torch.bfloat16 if dev.type == "cuda" else p.dtype)
    strategy = [("fsdp", {"atorch_wrap_cls": (MixtralDecoderLayer,), "atorch_ignored_cls": (Grouped_GEMM_MoE,),
                          "sync_module_states": True}),
                ("amp_native", {"dtype": torch.bfloat16})]
    ok, res, _ = auto_accelerate(model, torch.optim.AdamW, loss_func=lambda b, o: o[0], optim_args={"lr": 3e-4},
                                 load_strategy=strategy)
    assert ok
    eopt = BF16Optimizer(torch.optim.AdamW(expert_params, lr=3e-4)) if dev.type == "cuda" else \
        torch.optim.AdamW(expert_params, lr=3e-4)
    ids = torch.randint(0, cfg.vocab_size, (1, seq), device=dev)

    def step(i):
        res.optim.zero_grad()
        eopt.zero_grad()
        loss = res.model(input_ids=ids, labels=ids, return_logits=False)[0]
        loss.backward()
        res.optim.step()
        eopt.step()
        return loss
    ms = timed_steps(step, a.steps, a.warmup, dev)
    tokens = world * seq * a.steps
    report(rank, {"metric": "tokens/sec Mixtral-style MoE EP (device-timed, max over ranks)",
                  "value": round(tokens / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
                  "ms_per_step": round(ms / a.steps, 2), "dtype": "fp8 experts / bf16 rest" if a.fp8 else "bf16",
                  "config": {"layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size, "experts": cfg.num_experts,
                             "top_k": cfg.top_k, "expert_ffn": cfg.expert_intermediate_size, "seq_len": seq,
                             "dispatcher": disp, "capacity_factor": cfg.capacity_factor,
                             "parallelism": f"ep{world} + fsdp{world}"}})


if __name__ == "__main__":
    main()
