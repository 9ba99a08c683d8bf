"""Tensor / pipeline / expert / data parallelism on 2-4 GPUs over NCCL against single-GPU math, and the
tiny variants of the hybrid, MoE and local-SGD benchmark drivers on the GPU kernels."""
import glob

import pytest
import torch
import torch.nn as nn

from tests.dist_utils import run_distributed

pytestmark = pytest.mark.gpu
NGPU = torch.cuda.device_count()
WORLD = 8 if NGPU >= 8 else 4 if NGPU >= 4 else 2   # expert- and data-parallel tests use every GPU of the machine


# --------------------------------------------------------------------------------------- tensor parallel
def _tp_llama(rank, world):
    from atorch_b200.auto import auto_accelerate
    from atorch_b200.models.llama import LlamaConfig, LlamaModel
    from atorch_b200.modules.distributed_modules import ColumnParallelLinear, RowParallelLinear

    dev = torch.device("cuda", rank)
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=256)
    ref = LlamaModel(cfg).to(dev).bfloat16()
    ids = torch.randint(0, 512, (2, 256), device=dev)
    ref_loss, _ = ref(ids, labels=ids)
    ref_loss.backward()
    model = LlamaModel(cfg).to(dev).bfloat16()
    model.load_state_dict(ref.state_dict())
    ok, res, _ = auto_accelerate(model, load_strategy=[("parallel_mode", ([("tensor", world)], None)),
                                                       ("tensor_parallel", None)])
    assert ok
    m = res.model
    assert isinstance(m.layers[0].qkv_proj, ColumnParallelLinear) and isinstance(m.layers[0].down_proj, RowParallelLinear)
    loss, _ = m(ids, labels=ids)
    assert abs(loss.item() - ref_loss.item()) < 3e-2, (loss.item(), ref_loss.item())
    loss.backward()
    # a replicated parameter (final norm weight) gets the same gradient as on one GPU
    g, g_ref = m.norm.weight.grad.float(), ref.norm.weight.grad.float()
    assert torch.allclose(g, g_ref, rtol=5e-2, atol=5e-2 * g_ref.abs().max().item())


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_tensor_parallel_llama_matches_single_gpu():
    run_distributed(_tp_llama, world=2, backend="nccl", timeout=300)


# ------------------------------------------------------------------------------------- pipeline parallel
def _run_pipe(rank, world, vpp, sche, out_file):
    from atorch_b200.distributed import distributed as D
    from atorch_b200.pipeline_parallel.pipe_module import PipeModuleConfig, make_pipe_module
    from atorch_b200.pipeline_parallel.pipe_schedule import make_pipe_schedule_from_pipe_module
    from tests.test_pipeline_cpu import _Chunk

    dev = torch.device("cuda", rank)
    D.create_parallel_group(([("pipe", world)], None))

    def provider(model_config, layer_num, pre_process, post_process, start_layer_idx):
        return _Chunk(layer_num, pre_process, post_process, start_layer_idx).to(dev)

    cfg = PipeModuleConfig(total_layer_num=4, virtual_pp_size=vpp, sche_name=sche, n_microbatches=4, auto_ddp=False)
    pm = make_pipe_module(model_provider=provider, loss_func=lambda o, t: ((o - t) ** 2).mean(), config=cfg)
    sched = make_pipe_schedule_from_pipe_module(pm, cfg)
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(8, 8, generator=g).to(dev), torch.randn(8, 8, generator=g).to(dev)
    first = pm.stage_ids[0] == 0
    last = (pm.num_stages - 1) in pm.stage_ids
    if first and last:
        loss = sched.step(x, target=y)
    elif first:
        loss = sched.step(x)
    elif last:
        loss = sched.step(target=y)
    else:
        loss = sched.step()
    grads = {}
    for m, sid in zip(pm.stage_modules, pm.stage_ids):
        for i, l in enumerate(m.layers):
            grads[(sid, i)] = l.weight.grad.cpu().clone()
    torch.save({"loss": None if loss is None else float(loss), "grads": grads, "ids": pm.stage_ids},
               f"{out_file}.{rank}")


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_pipeline_schedules_match_single_process_nccl(tmp_path):
    from tests.test_pipeline_cpu import _reference

    ref_loss, ref_grads = _reference()
    for vpp, sche in ((1, "Schedule1F1B"), (2, "ScheduleInterleaved1F1B")):
        f = str(tmp_path / f"p_{vpp}_{sche}")
        run_distributed(_run_pipe, world=2, args=(vpp, sche, f), backend="nccl", timeout=300)
        per = 4 // (2 * vpp)
        seen_loss = False
        for r in range(2):
            d = torch.load(f"{f}.{r}")
            if d["loss"] is not None:
                assert abs(d["loss"] - ref_loss) < 1e-4
                seen_loss = True
            for (sid, i), gr in d["grads"].items():
                assert torch.allclose(gr, ref_grads[sid * per + i], atol=1e-4), (sche, sid, i)
        assert seen_loss


# --------------------------------------------------------------------------------------- expert parallel
def _ep(rank, world, dispatcher):
    from atorch_b200.distributed import distributed as D
    from atorch_b200.modules.moe import Grouped_GEMM_MoE
    from tests.test_moe_cpu import _dense_moe

    dev = torch.device("cuda", rank)
    D.create_parallel_group(([("expert", world)], None))
    torch.manual_seed(3)
    H, F, NE = 256, 512, max(4, world)
    full = Grouped_GEMM_MoE(H, F, 0.0, num_experts=NE, topk=2, use_swiglu=True)
    moe = Grouped_GEMM_MoE(H, F, 0.0, num_experts=NE, topk=2, use_swiglu=True, use_expert_parallelism=True,
                           token_dispatcher_type=dispatcher).to(dev).bfloat16()
    E = moe.num_local_experts
    with torch.no_grad():
        moe.w1.copy_(full.w1[rank * E:(rank + 1) * E])
        moe.w2.copy_(full.w2[rank * E:(rank + 1) * E])
    g = torch.Generator().manual_seed(10 + rank)
    x = (0.5 * torch.randn(64, H, generator=g)).to(dev).bfloat16().requires_grad_()
    logits = torch.randn(64, NE, generator=g)
    w, idx = torch.softmax(logits, -1).topk(2, -1)
    if dispatcher == "PeerMemory":
        assert moe.peer_exchange, "the peer-memory dispatcher was expected to be active"
    probs = w.to(dev).bfloat16().requires_grad_()
    y = moe(x, probs, idx.to(dev))
    full_bf = full.to(dev).bfloat16().float()
    xr = x.detach().float().requires_grad_()
    pr = probs.detach().float().requires_grad_()
    ref = _dense_moe(full_bf, xr, pr, idx.to(dev))
    err = (y.float() - ref).abs().max().item()
    assert err < 5e-2 * max(1.0, ref.abs().max().item()), (dispatcher, err)
    gout = torch.randn(y.shape, generator=torch.Generator().manual_seed(99 + rank)).to(dev)
    (y.float() * gout).sum().backward()
    (ref * gout).sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad.float()).all() and moe.w1.grad is not None
    gx_err = (x.grad.float() - xr.grad).abs().max().item()
    assert gx_err < 6e-2 * max(1.0, xr.grad.abs().max().item()), (dispatcher, "dx", gx_err)
    if probs.grad is not None:
        gp_err = (probs.grad.float() - pr.grad).abs().max().item()
        assert gp_err < 6e-2 * max(1.0, pr.grad.abs().max().item()), (dispatcher, "dprobs", gp_err)
    # expert weight gradients: every rank holds its own experts; compare with the dense gradient summed over
    # the ranks' tokens (all-reduce of the reference, which saw only this rank's tokens)
    gw = full_bf.w1.grad.clone()
    torch.distributed.all_reduce(gw)
    mine = gw[rank * E:(rank + 1) * E]
    gw_err = (moe.w1.grad.float() - mine).abs().max().item()
    assert gw_err < 6e-2 * max(1.0, mine.abs().max().item()), (dispatcher, "dw1", gw_err)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("dispatcher", ["PeerMemory", "AllToAll", "AllGather"])
def test_expert_parallel_matches_dense(dispatcher):
    run_distributed(_ep, world=WORLD, args=(dispatcher,), backend="nccl", timeout=300)


# ------------------------------------------------------------------------------------------ data parallel
def _ddp(rank, world, out_file):
    """Own bucketed DDP (all-reduce kernel over symmetric memory on NVSwitch systems) on fp32 gradients."""
    from atorch_b200.parallel.ddp import DistributedDataParallel
    from tests.test_fsdp_cpu import make_data, make_mlp

    dev = torch.device("cuda", rank)
    m = DistributedDataParallel(make_mlp().to(dev), bucket_cap_mb=0.5)
    assert m.symm is not None or world > 8, "the symmetric-memory all-reduce path was expected to be active"
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3)
    for x, y in make_data(rank, steps=8):
        opt.zero_grad()
        nn.functional.cross_entropy(m(x.to(dev)), y.to(dev)).backward()
        opt.step()
    if m.symm is not None:
        m.symm.check()
    if rank == 0:
        torch.save({k: v.cpu() for k, v in m.state_dict().items()}, out_file)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_ddp_own_allreduce_matches_single_process(tmp_path):
    from tests.test_fsdp_cpu import make_data, make_mlp

    f = str(tmp_path / "ddp.pt")
    run_distributed(_ddp, world=WORLD, args=(f,), backend="nccl", timeout=300)
    sd = torch.load(f)
    m = make_mlp()
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3)
    for parts in zip(*[make_data(r, steps=8) for r in range(WORLD)]):
        opt.zero_grad()
        (sum(nn.functional.cross_entropy(m(x), y) for x, y in parts) / WORLD).backward()
        opt.step()
    for k, v in m.state_dict().items():
        assert torch.allclose(sd[k], v, atol=2e-4, rtol=2e-3), k


# -------------------------------------------------------------------------- benchmark drivers, tiny configs
def _moe(rank, world, fp8):
    from atorch_b200.benchmarks import moe_bench

    moe_bench.main(["--tiny", "--fp8", str(fp8), "--steps", "2", "--warmup", "1"])


def _lsgd(rank, world, H):
    from atorch_b200.benchmarks import local_sgd_bench

    local_sgd_bench.main(["--tiny", "--H", str(H), "--windows", "1"])


def _hybrid(rank, world, out, tp, pp):
    from atorch_b200.benchmarks import hybrid_bench

    losses = hybrid_bench.main(["--tiny", "--tp", str(tp), "--pp", str(pp), "--micro-batches", "4", "--steps", "4",
                                "--warmup", "0"])
    if losses:
        torch.save(losses, f"{out}.{rank}")


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fp8", [0, 1])
def test_moe_bench_tiny_expert_parallel_nccl(fp8):
    run_distributed(_moe, world=min(NGPU, 4), args=(fp8,), backend="nccl", timeout=300)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("H", [2, 0])
def test_local_sgd_bench_tiny_nccl(H):
    run_distributed(_lsgd, world=min(NGPU, 4), args=(H,), backend="nccl", timeout=300)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_hybrid_bench_tiny_nccl(tmp_path):
    tp, pp = (2, 2) if NGPU >= 4 else (2, 1)
    world = 8 if NGPU >= 8 else (4 if NGPU >= 4 else 2)
    out = str(tmp_path / "h")
    run_distributed(_hybrid, world=world, args=(out, tp, pp), backend="nccl", timeout=400)
    files = glob.glob(out + ".*")
    assert files
    losses = torch.load(files[0])
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses


# ------------------------------------------------- tensor-parallel linears fused with their collectives
def _tp_fused(rank, world):
    """all-gather -> GEMM and GEMM -> reduce-scatter (ops/tp_fused.py) against torch.distributed collectives
    around a plain matmul, forward and backward, twice in a row (buffers and flags are reused)."""
    import torch.distributed as dist

    from atorch_b200 import _lib
    from atorch_b200.ops import tp_fused

    dev = torch.device("cuda", rank)
    assert tp_fused.available(dist.group.WORLD)
    rows, K, N = 512, 384, 640
    S = rows * world
    for it in range(2):
        g = torch.Generator().manual_seed(7 + 13 * rank + it)
        x_loc = (0.5 * torch.randn(rows, K, generator=g)).to(dev).bfloat16().requires_grad_()
        gw = torch.Generator().manual_seed(1000 + it)
        w = (0.05 * torch.randn(N, K, generator=gw)).to(dev).bfloat16().requires_grad_()
        # ---- all-gather -> GEMM
        y = tp_fused.allgather_linear(x_loc, w, dist.group.WORLD)
        xs = [torch.empty_like(x_loc) for _ in range(world)]
        dist.all_gather(xs, x_loc.detach())
        x_full = torch.cat(xs).float()
        ref = x_full @ w.detach().float().t()
        assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2), (it, (y.float() - ref).abs().max())
        gy = torch.randn(S, N, generator=torch.Generator().manual_seed(55 + rank + it)).to(dev).bfloat16()
        y.backward(gy)
        dx_full = gy.float() @ w.detach().float()                       # every rank's contribution to all rows
        dist.all_reduce(dx_full)
        dx_ref = dx_full[rank * rows:(rank + 1) * rows]
        assert torch.allclose(x_loc.grad.float(), dx_ref, rtol=3e-2, atol=3e-2 * dx_ref.abs().max().item()), it
        dw_ref = gy.float().t() @ x_full
        assert torch.allclose(w.grad.float(), dw_ref, rtol=3e-2, atol=3e-2 * dw_ref.abs().max().item()), it
        # ---- GEMM -> reduce-scatter (row-parallel: every rank holds its own slice of the features)
        x2 = (0.5 * torch.randn(S, K, generator=g)).to(dev).bfloat16().requires_grad_()
        w2 = (0.05 * torch.randn(N, K, generator=g)).to(dev).bfloat16().requires_grad_()
        y2 = tp_fused.linear_reduce_scatter(x2, w2, dist.group.WORLD)
        part = x2.detach().float() @ w2.detach().float().t()
        dist.all_reduce(part)
        ref2 = part[rank * rows:(rank + 1) * rows]
        assert torch.allclose(y2.float(), ref2, rtol=2e-2, atol=3e-2), (it, (y2.float() - ref2).abs().max())
        gy2 = torch.randn(rows, N, generator=torch.Generator().manual_seed(77 + rank + it)).to(dev).bfloat16()
        y2.backward(gy2)
        gs = [torch.empty_like(gy2) for _ in range(world)]
        dist.all_gather(gs, gy2)
        gfull = torch.cat(gs).float()
        dx2_ref = gfull @ w2.detach().float()
        assert torch.allclose(x2.grad.float(), dx2_ref, rtol=3e-2, atol=3e-2 * dx2_ref.abs().max().item()), it
        dw2_ref = gfull.t() @ x2.detach().float()
        assert torch.allclose(w2.grad.float(), dw2_ref, rtol=3e-2, atol=3e-2 * dw2_ref.abs().max().item()), it
    torch.cuda.synchronize()
    _lib.check_status(dev)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_tp_linears_fused_with_collectives():
    run_distributed(_tp_fused, world=min(NGPU, 4) if NGPU != 3 else 2, backend="nccl", timeout=300)


def test_allgather_gemm_gate_times_out_cleanly():
    """One GPU, no peer: an arrival flag that nothing sets. The GEMM's producer gives up after the (shortened)
    limit, the kernel drains and frees its tensor memory, the status word reports a peer timeout, and the
    next ordinary GEMM works."""
    import ctypes

    from atorch_b200 import _lib, ops

    L = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    a = torch.randn(512, 256, device=dev, dtype=torch.bfloat16)
    b = torch.randn(256, 256, device=dev, dtype=torch.bfloat16)
    y = torch.zeros(512, 256, device=dev, dtype=torch.bfloat16)
    flags = torch.zeros(2, dtype=torch.int32, device=dev)
    flags[0] = 1                                            # shard 0 arrived, shard 1 never does
    assert L.atb_set_gate_wait_ns(ctypes.c_ulonglong(50_000_000)) == 0
    try:
        rc = L.atb_gemm_bf16_2cta_fused(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(y), ctypes.c_int(512), ctypes.c_int(256), ctypes.c_int(256),
            ctypes.c_longlong(256), ctypes.c_longlong(256), ctypes.c_longlong(256), ctypes.c_int(0), ctypes.c_int(0),
            ctypes.c_float(1.0), _lib.ptr(flags), ctypes.c_uint(1), ctypes.c_int(256), ctypes.c_int(0), None,
            ctypes.c_int(0), ctypes.c_int(0), _lib.stream_ptr(), _lib.ptr(_lib.status_word(dev)))
        assert rc == 0
        with pytest.raises(_lib.KernelError):
            _lib.check_status(dev)
    finally:
        assert L.atb_set_gate_wait_ns(ctypes.c_ulonglong(2_000_000_000)) == 0
    ref = a.float() @ b.float().t()
    out = ops.gemm(a, b)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-1)


# --------------------------------------------- row-sharded weight: all-gather fused into the consuming GEMM
def _sharded_weight(rank, world):
    """ops.tp_fused.sharded_weight_linear (weight all-gather -> GEMM, weight-gradient GEMM -> reduce-scatter)
    against the torch.distributed form, twice in a row; every rank has its own input (data parallel)."""
    import torch.distributed as dist

    from atorch_b200 import _lib
    from atorch_b200.ops import tp_fused

    dev = torch.device("cuda", rank)
    rows, K, M = 256, 384, 640
    N = rows * world
    assert tp_fused.sharded_weight_available(dist.group.WORLD, rows, N, K)
    for it in range(2):
        gw = torch.Generator().manual_seed(500 + it)
        w_full = (0.05 * torch.randn(N, K, generator=gw)).bfloat16()
        w_shard = w_full[rank * rows:(rank + 1) * rows].to(dev).requires_grad_()
        g = torch.Generator().manual_seed(11 + 17 * rank + it)
        x = (0.5 * torch.randn(M, K, generator=g)).to(dev).bfloat16().requires_grad_()
        y = tp_fused.sharded_weight_linear(x, w_shard, dist.group.WORLD)
        assert type(y.grad_fn).__name__ == "_ShardedWeightLinearBackward"
        ref = x.detach().float() @ w_full.to(dev).float().t()
        assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2), (it, (y.float() - ref).abs().max())
        gy = torch.randn(M, N, generator=g).to(dev).bfloat16()
        y.backward(gy)
        dx_ref = gy.float() @ w_full.to(dev).float()
        assert torch.allclose(x.grad.float(), dx_ref, rtol=3e-2, atol=3e-2 * dx_ref.abs().max().item()), it
        dw = gy.float().t() @ x.detach().float()
        dist.all_reduce(dw)
        dw_ref = dw[rank * rows:(rank + 1) * rows]
        assert torch.allclose(w_shard.grad.float(), dw_ref, rtol=3e-2, atol=3e-2 * dw_ref.abs().max().item()), it
    torch.cuda.synchronize()
    _lib.check_status(dev)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_sharded_weight_linear_fused_with_collectives():
    run_distributed(_sharded_weight, world=min(NGPU, 4) if NGPU != 3 else 2, backend="nccl", timeout=300)


# ------------------------------------------------- sequence parallel attention on the flash kernels (ring, Ulysses)
def _ring_flash(rank, world):
    """Ring attention with the flash kernels per chunk and K/V chunks pulled over peer memory, causal and full,
    forward and backward, twice in a row (buffers are reused), against dense attention on the whole sequence."""
    import torch.distributed as dist

    from atorch_b200 import _lib
    from atorch_b200.ops import attention_reference, ring_flash
    from atorch_b200.parallel.sequence_parallel import UlyssesAttention, ring_attention

    dev = torch.device("cuda", rank)
    B, S_loc, H, D = 2, 256, 4, 128
    S = S_loc * world
    for it, causal in enumerate((True, False, True)):
        g = torch.Generator().manual_seed(40 + it)
        full = [(0.5 * torch.randn(B, S, H, D, generator=g)).to(dev).bfloat16() for _ in range(3)]
        gy = torch.randn(B, S, H, D, generator=g).to(dev).bfloat16()
        sl = slice(rank * S_loc, (rank + 1) * S_loc)
        q, k, v = (t[:, sl].clone().requires_grad_() for t in full)
        assert ring_flash.available(q, k, v, dist.group.WORLD)
        out = ring_attention(q, k, v, dist.group.WORLD, causal=causal)
        assert type(out.grad_fn).__name__ == "_RingFlashBackward"
        out.backward(gy[:, sl])
        rq, rk, rv = (t.float().requires_grad_() for t in full)
        ref = attention_reference(rq, rk, rv, causal=causal)
        ref.backward(gy.float())
        torch.cuda.synchronize()
        _lib.check_status(dev)
        assert torch.allclose(out.float(), ref[:, sl], rtol=2e-2, atol=2e-2), (it, (out.float() - ref[:, sl]).abs().max())
        for name, a, b in (("q", q, rq), ("k", k, rk), ("v", v, rv)):
            gb = b.grad[:, sl]
            err = (a.grad.float() - gb).abs().max().item()
            assert err < 3e-2 * (gb.abs().max().item() + 1e-6), (it, name, err)
        if causal:
            # load-balanced layout: rank r holds pieces r and 2W-1-r of the sequence
            zq, zk, zv = (ring_flash.zigzag_shard(t, rank, world).clone().requires_grad_() for t in full)
            zo = ring_attention(zq, zk, zv, dist.group.WORLD, causal=True, layout="zigzag")
            zo.backward(ring_flash.zigzag_shard(gy, rank, world))
            torch.cuda.synchronize()
            _lib.check_status(dev)
            zref = ring_flash.zigzag_shard(ref, rank, world)
            assert torch.allclose(zo.float(), zref, rtol=2e-2, atol=2e-2), (it, (zo.float() - zref).abs().max())
            for name, a, b in (("q", zq, rq), ("k", zk, rk), ("v", zv, rv)):
                gb = ring_flash.zigzag_shard(b.grad, rank, world)
                err = (a.grad.float() - gb).abs().max().item()
                assert err < 3e-2 * (gb.abs().max().item() + 1e-6), (it, "zigzag", name, err)
        # Ulysses on the same data: heads scattered, sequence gathered, flash kernels locally
        ul = UlyssesAttention(causal=causal)
        ul.set_sp(world, rank, dist.group.WORLD)
        q2, k2, v2 = (t[:, sl].clone().requires_grad_() for t in full)
        o2 = ul(q2, k2, v2)
        assert torch.allclose(o2.float(), ref[:, sl], rtol=2e-2, atol=2e-2), it
        o2.backward(gy[:, sl])
        for name, a, b in (("q", q2, rq), ("k", k2, rk), ("v", v2, rv)):
            gb = b.grad[:, sl]
            assert (a.grad.float() - gb).abs().max().item() < 3e-2 * (gb.abs().max().item() + 1e-6), (it, name)


@pytest.mark.skipif(NGPU < 2, reason="needs 2 GPUs")
def test_ring_attention_on_flash_kernels_over_peer_memory():
    run_distributed(_ring_flash, world=min(NGPU, 4) if NGPU != 3 else 2, backend="nccl", timeout=300)
