"""Hybrid-parallel Llama benchmark: tensor parallel (optionally with sequence parallel) x pipeline parallel
(1F1B) x sharded data parallel, AGD optimizer.

    torchrun --nproc-per-node 8 -m atorch_b200.benchmarks.hybrid_bench --tp 2 --pp 2 [--tiny]

Llama-2 13B (40 layers, hidden 5120, 40 heads, FFN 13824), seq 4096, micro-batch 1, 8 micro-batches per step.
Every pipeline stage chunk is tensor-parallelised (column / row linears, vocabulary-parallel embedding), wrapped
by the sharded engine over the ``data`` group with per-layer recomputation, and driven by the 1F1B schedule.
"""
from __future__ import annotations

import json
import argparse

import torch
import torch.nn as nn

from atorch_b200 import ops
from atorch_b200.benchmarks.common import reference_unavailable, report, setup, timed_steps
from atorch_b200.distributed import distributed as D
from atorch_b200.models.llama import LlamaConfig, LlamaDecoderLayer, RMSNorm, causal_lm_loss
from atorch_b200.parallel.fsdp import FSDP, FusedShardedOptimizer
from atorch_b200.modules.distributed_modules.mappings import gather_from_group, scatter_to_group
from atorch_b200.parallel.tensor_parallel import (apply_tensor_parallel, mark_sequence_parallel_replicated,
                                                  sync_sequence_parallel_grads)
from atorch_b200.pipeline_parallel.pipe_module import PipeModuleConfig, make_pipe_module
from atorch_b200.pipeline_parallel.pipe_schedule import make_pipe_schedule_from_pipe_module


class LlamaChunk(nn.Module):
    """Layers [start, start + n) of a Llama model, with the embedding on the first chunk and the final norm
    + LM head on the last."""

    def __init__(self, cfg: LlamaConfig, layer_num: int, pre: bool, post: bool, start: int, sp: bool = False):
        super().__init__()
        self.cfg = cfg
        self.sp = sp          # activations between the tensor-parallel blocks are sharded along the sequence
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size) if pre else None
        self.layers = nn.ModuleList([LlamaDecoderLayer(cfg, start + i) for i in range(layer_num)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps) if post else None
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False) if post else None
        self._rope = {}
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=cfg.initializer_range)

    def forward(self, x):
        tp_group = D.parallel_group("tensor") if self.sp else None
        if self.embed_tokens is not None:
            h = self.embed_tokens(x)
            if self.sp:
                h = scatter_to_group(h, tp_group, dim=1)          # keep this rank's part of the sequence
        else:
            h = x
        S = h.shape[1] * ((D.parallel_group_size("tensor") or 1) if self.sp else 1)
        key = (S, str(x.device))
        if key not in self._rope:
            self._rope = {key: ops.rope_tables(S, self.cfg.head_dim, self.cfg.rope_theta, x.device)}
        cos, sin = self._rope[key]
        for l in self.layers:
            h = l(h, cos, sin)
        if self.lm_head is not None:
            h = self.norm(h)
            if self.sp:
                # the head is replicated over the tensor group (every rank computes the same logits), so the
                # backward of this gather is a split, not a reduce-scatter
                h = gather_from_group(h, tp_group, dim=1)
            h = ops.linear(h, self.lm_head.weight)
        return h


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--micro-batches", type=int, default=8)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--sp", type=int, default=1, help="sequence parallelism inside the tensor-parallel group")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    a = ap.parse_args(argv)
    if a.impl == "reference":
        reference_unavailable("not wired: the reference has no single entry point for TP2 + sequence parallel + PP2 + DP2; its nearest runnable piece (PP x DDP with AGD through make_pipe_module, examples/llama2/train_llama2_with_pp.py) was not brought up on this image")
        return
    rank, world, dev = setup()
    dp = world // (a.tp * a.pp)
    D.create_parallel_group(([("tensor", a.tp), ("pipe", a.pp), ("data", dp)], None))
    cfg = LlamaConfig.tiny(num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=4) if a.tiny \
        else LlamaConfig.llama2_13b()
    if a.layers:
        cfg.num_hidden_layers = a.layers
    sp = bool(a.sp) and a.tp > 1
    seq = 64 if a.tiny else 4096
    bf16 = dev.type == "cuda"

    def provider(model_config, layer_num, pre_process, post_process, start_layer_idx):
        torch.manual_seed(1000 + start_layer_idx)                 # same weights on all tensor / data ranks of a stage
        with torch.device(dev):
            chunk = LlamaChunk(cfg, layer_num, pre_process, post_process, start_layer_idx, sp=sp)
        if a.tp > 1:
            apply_tensor_parallel(chunk, {"sequence_parallel": sp})
            if sp:
                mark_sequence_parallel_replicated(chunk, (RMSNorm,))
        return FSDP(chunk, wrap_cls=(LlamaDecoderLayer,), process_group=D.parallel_group("data"),
                    param_dtype=torch.bfloat16 if bf16 else None, checkpoint_units=True, device=dev)

    def loss_fn(logits, labels):
        return causal_lm_loss(logits, labels)
    pcfg = PipeModuleConfig(total_layer_num=cfg.num_hidden_layers, sche_name="Schedule1F1B",
                            n_microbatches=a.micro_batches, auto_ddp=False)
    pm = make_pipe_module(model_provider=provider, loss_func=loss_fn, config=pcfg)
    sched = make_pipe_schedule_from_pipe_module(pm, pcfg)
    optims = [FusedShardedOptimizer(m.engine, "agd", lr=3e-4) for m in pm.stage_modules]
    first, last = 0 in pm.stage_ids, (pm.num_stages - 1) in pm.stage_ids
    g = torch.Generator().manual_seed(7 + (D.parallel_rank("data") or 0))
    ids = torch.randint(0, cfg.vocab_size, (a.micro_batches, seq), generator=g).to(dev)
    losses = []

    def step(i):
        for o in optims:
            o.zero_grad()
        if first and last:
            l = sched.step(ids, target=ids)
        elif first:
            l = sched.step(ids)
        elif last:
            l = sched.step(target=ids)
        else:
            l = sched.step()
        if sp:
            for m in pm.stage_modules:
                sync_sequence_parallel_grads(m)
        for o in optims:
            o.step()
        if l is not None:
            losses.append(float(l))
        return l
    ms = timed_steps(step, a.steps, a.warmup, dev)
    tokens = dp * a.micro_batches * seq * a.steps
    rec = {"metric": "tokens/sec hybrid TP x PP x DP (device-timed, max over ranks)",
           "value": round(tokens / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
           "ms_per_step": round(ms / a.steps, 2),
           "config": {"model": "tiny" if a.tiny else "llama2-13b", "layers": cfg.num_hidden_layers, "tp": a.tp,
                      "sequence_parallel": sp, "pp": a.pp, "dp": dp, "seq_len": seq,
                      "micro_batches": a.micro_batches, "schedule": "1F1B", "optimizer": "AGD lr 3e-4"}}
    if last and (D.parallel_rank("tensor") or 0) == 0 and (D.parallel_rank("data") or 0) == 0:
        rec["losses"] = [round(x, 4) for x in losses]
        print("LAST_STAGE " + json.dumps(rec), flush=True)
    report(rank, rec)
    return losses


if __name__ == "__main__":
    main()
