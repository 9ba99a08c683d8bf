"""Sharded engine and DDP on CPU/gloo (world 2): loss curves of DDP and FSDP agree with a single
process on the union batch; full state dicts round-trip; the toy config of the benchmark suite
(4-layer MLP 256-512-512-512-10, AdamW 1e-3, 20 steps, batch 16 per rank) runs through auto_accelerate."""
import copy

import torch
import torch.nn as nn

from tests.dist_utils import run_distributed


def make_mlp():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(256, 512), nn.ReLU(), nn.Linear(512, 512), nn.ReLU(), nn.Linear(512, 512), nn.ReLU(),
                      nn.Linear(512, 10))
    for p in m.parameters():
        if p.dim() > 1:
            nn.init.normal_(p, std=0.02)
    return m


def make_data(rank, steps=20, per_rank=16):
    g = torch.Generator().manual_seed(1000 + rank)
    return [(torch.randn(per_rank, 256, generator=g), torch.randint(0, 10, (per_rank,), generator=g))
            for _ in range(steps)]


def loss_func(batch, out):
    return nn.functional.cross_entropy(out, batch[1])


def _train(rank, world, strategy, tmp):
    from atorch_b200.auto import auto_accelerate

    ok, res, _ = auto_accelerate(make_mlp(), torch.optim.AdamW, loss_func=loss_func, optim_args={"lr": 1e-3},
                                 load_strategy=strategy)
    assert ok
    losses = []
    for batch in make_data(rank):
        res.optim.zero_grad()
        loss = res.loss_func(batch, res.model(batch[0]))
        loss.backward()
        res.optim.step()
        losses.append(loss.item())
    sd = res.model.state_dict()
    if rank == 0:
        torch.save({"losses": losses, "sd": {k: v.clone() for k, v in sd.items()}}, tmp)


def _single(tmp):
    m = make_mlp()
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3)
    d0, d1 = make_data(0), make_data(1)
    losses0 = []
    for (x0, y0), (x1, y1) in zip(d0, d1):
        opt.zero_grad()
        l0 = nn.functional.cross_entropy(m(x0), y0)
        l1 = nn.functional.cross_entropy(m(x1), y1)
        ((l0 + l1) / 2).backward()
        opt.step()
        losses0.append(l0.item())
    return losses0, m.state_dict()


def test_ddp_and_fsdp_match_single_process(tmp_path):
    ref_losses, ref_sd = _single(None)
    for name, strategy in [
        ("ddp", ["parallel_mode"]),
        ("fsdp", ["parallel_mode", ("fsdp", {"atorch_wrap_cls": (nn.Linear,)})]),
        ("fsdp_size", ["parallel_mode", ("fsdp", {"atorch_size_based_min_num_params": 1000})]),
        ("zero2", ["parallel_mode", ("zero2", {"atorch_wrap_cls": (nn.Linear,)})]),
        ("zero1", ["parallel_mode", "zero1"]),
        ("fsdp_ckpt", ["parallel_mode", ("fsdp", {"atorch_wrap_cls": (nn.Linear,)}),
                       ("checkpoint", {"wrap_class": (nn.Linear,)})]),
    ]:
        f = str(tmp_path / f"{name}.pt")
        run_distributed(_train, world=2, args=(strategy, f))
        got = torch.load(f)
        assert max(abs(a - b) for a, b in zip(got["losses"], ref_losses)) < 2e-4, name
        for k, v in ref_sd.items():
            key = k if k in got["sd"] else "module." + k
            assert torch.allclose(got["sd"][key], v, atol=2e-5), (name, k)


def _hybrid(rank, world, tmp):
    from atorch_b200.auto import auto_accelerate
    from atorch_b200.parallel.fsdp import FSDP

    strategy = [("parallel_mode", ([("zero", 2), ("data", 2)], None)), ("fsdp", {"atorch_wrap_cls": (nn.Linear,)})]
    ok, res, _ = auto_accelerate(make_mlp(), torch.optim.AdamW, loss_func=loss_func, optim_args={"lr": 1e-3},
                                 load_strategy=strategy)
    assert ok and isinstance(res.model, FSDP)
    assert res.model.engine.world == 2 and res.model.engine.replicas == 2
    data = make_data(rank % 2)          # replicas see the same two shards of data as the 2-rank runs
    losses = []
    for batch in data[:5]:
        res.optim.zero_grad()
        loss = res.loss_func(batch, res.model(batch[0]))
        loss.backward()
        res.optim.step()
        losses.append(loss.item())
    if rank == 0:
        torch.save(losses, tmp)


def test_hybrid_shard_matches(tmp_path):
    ref_losses, _ = _single(None)
    f = str(tmp_path / "h.pt")
    run_distributed(_hybrid, world=4, args=(f,))
    got = torch.load(f)
    assert max(abs(a - b) for a, b in zip(got, ref_losses[:5])) < 2e-4


def _state_dict_roundtrip(rank, world):
    from atorch_b200.parallel.fsdp import FSDP, FusedShardedOptimizer

    m = make_mlp()
    ref = copy.deepcopy(m.state_dict())
    f = FSDP(m, wrap_cls=(nn.Linear,))
    sd = f.state_dict()
    for k, v in ref.items():
        assert torch.equal(sd[k], v)
    sd2 = {k: v + 1.0 for k, v in sd.items()}
    f.load_state_dict(sd2)
    sd3 = f.state_dict()
    for k in ref:
        assert torch.equal(sd3[k], sd2[k])
    opt = FusedShardedOptimizer(f.engine, "adamw", lr=1e-3)
    x = torch.randn(4, 256)
    f(x).sum().backward()
    n0 = f.clip_grad_norm_(0.5)
    assert torch.isfinite(n0)
    assert abs(f.engine.grad_norm().item() - min(0.5, n0.item())) < 1e-3
    opt.step()


def test_state_dict_and_clip():
    run_distributed(_state_dict_roundtrip, world=2)


def _frozen_odd(rank, world, device_type):
    """Odd-sized bias (alignment gaps, tail padding) and one frozen parameter: the sharded gradient norm
    equals the unsharded one and the frozen weights neither move nor decay."""
    from atorch_b200.auto import auto_accelerate

    dev = torch.device(device_type, rank) if device_type == "cuda" else torch.device("cpu")
    dtype_kw = [("amp_native", {"dtype": torch.bfloat16})] if device_type == "cuda" else []

    def make():
        torch.manual_seed(7)
        m = nn.Sequential(nn.Linear(24, 37), nn.Tanh(), nn.Linear(37, 13), nn.Tanh(), nn.Linear(13, 5))
        m[2].weight.requires_grad_(False)
        return m

    ok, res, _ = auto_accelerate(make(), torch.optim.AdamW, optim_args={"lr": 1e-2, "weight_decay": 0.1},
                                 load_strategy=["parallel_mode", ("fsdp", {"atorch_wrap_cls": (nn.Linear,)})] + dtype_kw)
    assert ok
    ref = make().to(dev)
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(world * 4, 24, generator=g) for _ in range(3)]
    frozen0 = ref[2].weight.detach().clone()
    opt = torch.optim.AdamW([p for p in ref.parameters() if p.requires_grad], lr=1e-2, weight_decay=0.1)
    tol = 5e-2 if device_type == "cuda" else 1e-5
    for x in xs:
        res.optim.zero_grad()
        res.model(x[rank * 4:(rank + 1) * 4].to(dev)).float().pow(2).mean().backward()
        norm = res.model.engine.grad_norm(2.0)
        opt.zero_grad()
        ref(x.to(dev)).pow(2).mean().backward()
        ref_norm = torch.sqrt(sum(p.grad.float().pow(2).sum() for p in ref.parameters() if p.grad is not None))
        assert torch.isfinite(norm)
        assert abs(norm.item() - ref_norm.item()) <= tol * max(1.0, ref_norm.item()), (norm.item(), ref_norm.item())
        res.optim.step()
        opt.step()
    sd = res.model.state_dict()
    assert torch.equal(sd["2.weight"].to(frozen0.device).to(frozen0.dtype), frozen0)
    for (n, p) in ref.named_parameters():
        assert torch.allclose(sd[n].to(p.device), p.detach().float(), atol=10 * tol, rtol=10 * tol), n


def test_fsdp_frozen_and_odd_sizes_gloo():
    run_distributed(_frozen_odd, world=2, args=("cpu",))
