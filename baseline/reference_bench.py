"""Reference arm of ``bench.py``: the unmodified reference framework, installed under
``baseline/_ref`` (``pip install --target baseline/_ref`` from a copy of the reference tree), driven
through its own public API and stock code path: ``atorch.init_distributed`` +
``atorch.auto.accelerate.auto_accelerate`` on a Hugging Face ``LlamaForCausalLM`` with the strategy
of its own example (examples/llama2/train_llama2_dummy_data.py:148-194: parallel_mode,
module_replace, fsdp{sync_module_states, limit_all_gathers, forward_prefetch,
atorch_wrap_cls=(LlamaDecoderLayer,)}, amp_native bf16, checkpoint{LlamaDecoderLayer, no_reentrant}).
Nothing of atorch_b200 is imported here. Same metric, config, timing rules and JSON line as the
framework's own arm, with ``"impl": "reference"``.
"""
from __future__ import annotations

import json
import os
import sys
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why[:300]}), flush=True)


def run(args, MODELS, PUBLISHED, ClockSampler, helpers=None) -> None:
    if not os.path.isdir(os.path.join(REF_DIR, "atorch")):
        return _unavailable("baseline/_ref/atorch is missing: the reference was not installed on this machine")
    # the repository root must not shadow the reference's `atorch` package
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    sys.path.insert(0, REF_DIR)
    try:
        import torch
        import atorch
        assert os.path.abspath(atorch.__file__).startswith(REF_DIR), atorch.__file__
        from atorch.auto.accelerate import auto_accelerate
        from atorch.common.util_func import data_to_device
        from transformers.models.llama.configuration_llama import LlamaConfig
        from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaForCausalLM
    except Exception as e:  # noqa
        return _unavailable(f"import of the reference failed: {type(e).__name__}: {e}")
    try:
        _run(args, MODELS, PUBLISHED, ClockSampler, torch, atorch, auto_accelerate, data_to_device, LlamaConfig,
             LlamaDecoderLayer, LlamaForCausalLM, helpers or {})
    except Exception as e:  # noqa
        traceback.print_exc()
        _unavailable(f"reference run failed: {type(e).__name__}: {str(e).splitlines()[0] if str(e) else ''}")


def _run(args, MODELS, PUBLISHED, ClockSampler, torch, atorch, auto_accelerate, data_to_device, LlamaConfig,
         LlamaDecoderLayer, LlamaForCausalLM, helpers):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ok = atorch.init_distributed("nccl", set_cuda_device_using_local_rank=True)
    assert ok, "atorch.init_distributed failed"
    rank = dist.get_rank()

    mc = MODELS[args.model]
    seq = args.seq or mc["max_position_embeddings"]
    cfg = LlamaConfig(vocab_size=mc["vocab_size"], hidden_size=mc["hidden_size"],
                      intermediate_size=mc["intermediate_size"], num_hidden_layers=mc["num_hidden_layers"],
                      num_attention_heads=mc["num_attention_heads"], num_key_value_heads=mc["num_key_value_heads"],
                      max_position_embeddings=mc["max_position_embeddings"], initializer_range=0.02)
    cfg._attn_implementation = "flash_attention_2"
    cfg.use_cache = False
    torch.manual_seed(1234)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg)
    loss_curve = getattr(args, "loss_curve", 0)
    if loss_curve:      # the same name-seeded weights as the other arm (plain tensor fills, nothing of its code)
        with torch.no_grad():
            for name, p in model.named_parameters():
                helpers["name_seeded_init_"](name, p)

    def loss_func(inputs, output):
        return output.loss

    # the example asks for a device mesh; with one process the reference cannot build a 0-D mesh
    # ("No `mesh_dim_names` found"), so the plain group form is used there
    strategy = [("parallel_mode", ([("data", world)], None, False, world > 1)), "module_replace",
                ("fsdp", {"sync_module_states": True, "limit_all_gathers": True, "forward_prefetch": True,
                          "atorch_wrap_cls": (LlamaDecoderLayer,)}),
                ("amp_native", {"dtype": torch.bfloat16}),
                ("checkpoint", {"wrap_class": (LlamaDecoderLayer,), "no_reentrant": True})]
    status, res, _ = auto_accelerate(model, optim_func=torch.optim.AdamW, dataset=None, loss_func=loss_func,
                                     prepare_input=data_to_device, model_input_format="unpack_dict",
                                     optim_args={"lr": 3e-4, "weight_decay": 0.01, "betas": (0.9, 0.999)},
                                     dataloader_args=None, load_strategy=strategy)
    assert status, "reference auto_accelerate returned status False"
    model, optim, prepare_input = res.model, res.optim, res.prepare_input
    B = args.mbs
    if loss_curve:
        losses = []
        for ids in helpers["loss_stream"](cfg.vocab_size, B, seq, rank, loss_curve):
            batch = {"input_ids": ids.to(dev), "labels": ids.to(dev)}
            optim.zero_grad()
            loss = res.loss_func(batch, model(**batch))
            loss.backward()
            optim.step()
            t = loss.detach().float().clone()
            if world > 1:
                dist.all_reduce(t)
            losses.append(float(t.item()) / world)
        if rank == 0:
            rec = {"impl": "reference", "n_gpus": world, "model": args.model, "seq_len": seq, "steps": loss_curve,
                   "loss_curve": losses}
            if getattr(args, "loss_out", None):
                json.dump(rec, open(args.loss_out, "w"))
            print(json.dumps({k: v for k, v in rec.items() if k != "loss_curve"} |
                             {"first": losses[0], "last": losses[-1]}), flush=True)
        if world > 1:
            dist.barrier()
        return
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    n_host = args.steps + args.warmup
    host = [torch.randint(0, cfg.vocab_size, (B, seq), generator=gen).pin_memory() for _ in range(n_host)]
    dev_batch = {"input_ids": host[0].to(dev), "labels": host[0].to(dev)}

    def step_device(i):
        optim.zero_grad()
        out = model(**dev_batch)
        loss = res.loss_func(dev_batch, out)
        loss.backward()
        optim.step()
        return loss

    def step_e2e(i):
        ids = host[i % n_host]
        batch = prepare_input({"input_ids": ids, "labels": ids}, dev)
        optim.zero_grad()
        out = model(**batch)
        loss = res.loss_func(batch, out)
        loss.backward()
        optim.step()
        return float(loss.item())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        last = None
        for i in range(steps):
            last = fn(i)
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), last

    for i in range(args.warmup):
        step_device(i)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, _ = timed(step_device, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    tokens = world * B * seq * args.steps
    value = tokens / (ms / 1e3)
    e2e = None
    if not args.no_e2e:
        for i in range(2):
            step_e2e(i)
        ms2, last_loss = timed(step_e2e, args.steps)
        e2e = {"value": round(tokens / (ms2 / 1e3), 1), "unit": "tokens/s", "h2d_bytes_per_step": B * seq * 8 * 2,
               "d2h_bytes_per_step": 4, "ms_per_step": round(ms2 / args.steps, 2), "last_loss": last_loss}
    if rank == 0:
        print(json.dumps({
            "metric": "tokens/sec/box (device-timed, max over ranks) Llama-2 7B FSDP", "value": round(value, 1),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / (PUBLISHED * world), 3) if args.model == "llama2-7b" else None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights", "impl": "reference",
            "config": {"model": args.model, "global_batch": world * B, "seq_len": seq,
                       "parallelism": f"fsdp{world}" if world > 1 else "single GPU (the reference drops fsdp at world size 1)",
                       "optimizer": "torch AdamW lr 3e-4", "activation_checkpointing": "per layer",
                       "l2": "not flushed: weights and optimizer state far exceed the 126 MB L2"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": 0,
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
            "reference_module": os.path.dirname(atorch.__file__)}), flush=True)
    if world > 1:
        dist.barrier()
    try:
        atorch.reset_distributed()
    except Exception:
        pass
