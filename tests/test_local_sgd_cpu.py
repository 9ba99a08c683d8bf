"""Local SGD on CPU/gloo: anomaly detector, reducers, outer optimizer averager vs a hand-rolled reference."""
import copy
import math

import torch
import torch.distributed as dist
import torch.nn as nn

from atorch_b200.local_sgd import (GTAConfig, LocalSGDConfig, OnlineDynamicEWMA, OuterOptimizerConfig,
                                   OuterOptimPeriodicModelAverager, StatefulPostLocalSGDOptimizer, sparsify)
from atorch_b200.local_sgd.reducers import GTAReducer, LinearReducer
from tests.dist_utils import run_distributed


def test_ewma_detects_spike_after_warmup():
    d = OnlineDynamicEWMA(alpha=0.1, warmup_steps=20, base_threshold=3)
    g = torch.Generator().manual_seed(0)
    for _ in range(50):
        x = 1.0 + 0.01 * torch.randn((), generator=g).item()
        assert not d.is_outlier(x)
        d.update(x)
    assert d.is_outlier(5.0) and not d.is_outlier(1.0)
    sd = d.state_dict()
    d2 = OnlineDynamicEWMA(alpha=0.1, warmup_steps=20, base_threshold=3)
    d2.load_state_dict(sd)
    assert d2.is_outlier(5.0) and abs(d2.get_mean() - d.get_mean()) < 1e-12


def test_sparsify():
    t = torch.arange(1, 101, dtype=torch.float32)
    s = sparsify(t.clone(), 0.1, "magnitude")
    assert (s != 0).sum() == 10 and s[-1] == 100
    torch.manual_seed(0)
    r = sparsify(torch.ones(10000), 0.3, "rescaled_random")
    assert abs(r.mean().item() - 1.0) < 0.05


def _reducers(rank, world):
    t = torch.full((8,), float(rank + 1))
    LinearReducer(None, normalize=True).reduce_tensor(t, weight=float(rank + 1))
    # sum w_i x_i / sum w_i with w = x = rank+1: (1 + 4) / 3
    assert torch.allclose(t, torch.full((8,), 5.0 / 3.0))
    t = torch.tensor([1.0, -1.0, 2.0, -3.0]) * (1 if rank == 0 else -1)
    t[0] = 1.0                                   # both agree on entry 0 only
    g = GTAReducer(None, consensus_method="sum", normalize=True)
    g.reduce_tensor(t)
    assert abs(t[0].item() - 1.0) < 1e-6         # agreed entry: average of the agreeing replicas
    a = torch.full((4,), float(rank))
    LinearReducer(None, normalize=False, weight_softmax_temperature=1.0).reduce_tensor(a, weight=float(rank))
    w = torch.softmax(torch.tensor([0.0, 1.0]), 0)
    assert torch.allclose(a, torch.full((4,), float(w[1])))


def test_reducers_gloo():
    run_distributed(_reducers, world=2)


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 4))


def _outer(rank, world, H, nesterov):
    model = _model()
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    avg = OuterOptimPeriodicModelAverager(
        local_sgd_config=LocalSGDConfig(local_sgd_sync_interval=H, local_sgd_warmup_steps=0),
        outer_optim_config=OuterOptimizerConfig(torch.optim.SGD, {"lr": 0.7, "momentum": 0.9, "nesterov": nesterov}))
    lopt = StatefulPostLocalSGDOptimizer(opt, avg)
    # hand-rolled reference: both replicas simulated in this process. As in the algorithm, every
    # replica snapshots its own "last synced" weights at the first averaging call.
    refs = [_model() for _ in range(world)]
    ropts = [torch.optim.SGD(m.parameters(), lr=0.1) for m in refs]
    synced, bufs = None, None
    outer_t = 0
    for step in range(2 * H + 1):
        for r in range(world):
            g = torch.Generator().manual_seed(100 * step + r)
            x, y = torch.randn(4, 8, generator=g), torch.randn(4, 4, generator=g)
            if r == rank:
                lopt.zero_grad()
                ((model(x) - y) ** 2).mean().backward()
            ropts[r].zero_grad()
            ((refs[r](x) - y) ** 2).mean().backward()
            ropts[r].step()
        if synced is None:
            synced = [[p.detach().clone() for p in m.parameters()] for m in refs]
            bufs = [torch.zeros_like(p) for p in synced[0]]
        if step % H == 0:
            for i in range(len(bufs)):
                pg = sum(synced[r][i] - list(refs[r].parameters())[i].detach() for r in range(world)) / world
                bufs[i] = pg.clone() if outer_t == 0 else 0.9 * bufs[i] + pg
                upd = pg + 0.9 * bufs[i] if nesterov else bufs[i]
                for r in range(world):
                    synced[r][i] -= 0.7 * upd
                    list(refs[r].parameters())[i].data.copy_(synced[r][i])
            outer_t += 1
        lopt.step()
        for p, q in zip(model.parameters(), refs[rank].parameters()):
            assert torch.allclose(p, q, atol=1e-5), step
    sd = lopt.state_dict()
    assert sd["averager"]["step"] == 2 * H + 1 and "outer_optimizer" in sd["averager"]
    lopt.load_state_dict(copy.deepcopy(sd))


def test_outer_nesterov_matches_reference():
    for H, nesterov in ((1, True), (3, True), (2, False)):
        run_distributed(_outer, world=2, args=(H, nesterov))


def _plain_average(rank, world):
    model = _model()
    with torch.no_grad():
        for p in model.parameters():
            p.add_(float(rank))
    avg = OuterOptimPeriodicModelAverager(local_sgd_config=LocalSGDConfig(local_sgd_sync_interval=1))
    before = [p.detach().clone() - float(rank) for p in model.parameters()]
    avg.average_parameters(model.parameters())
    for p, b in zip(model.parameters(), before):
        assert torch.allclose(p, b + 0.5, atol=1e-6)


def test_plain_average():
    run_distributed(_plain_average, world=2)


def _warmup_baseline(rank, world):
    """With warm-up steps the first outer step starts from the weights at the END of the warm-up: the
    pseudo-gradient of the first sync is only the drift of the local steps, never the warm-up progress.
    Checked against the outer Nesterov step written out by hand."""
    import torch.distributed as dist
    import torch.nn as nn

    from atorch_b200.auto import auto_accelerate
    from atorch_b200.local_sgd import LocalSGDConfig, OuterOptimizerConfig

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 8), nn.Tanh(), nn.Linear(8, 2))
    fs = {"atorch_wrap_cls": (nn.Linear,), "use_local_sgd": True,
          "local_sgd_config": LocalSGDConfig(local_sgd_sync_interval=2, local_sgd_warmup_steps=3),
          "outer_optim_config": OuterOptimizerConfig(torch.optim.SGD, {"lr": 0.7, "momentum": 0.9, "nesterov": True})}
    ok, res, _ = auto_accelerate(model, torch.optim.SGD, optim_args={"lr": 0.1},
                                 load_strategy=[("parallel_mode", ([("zero", 1), ("data", 2)], None)), ("fsdp", fs)])
    assert ok
    eng, lsgd = res.model.engine, res.model.engine.local_sgd
    g = torch.Generator().manual_seed(rank)
    base = None
    for step in range(4):
        res.optim.zero_grad()
        res.model(torch.randn(4, 8, generator=g)).pow(2).mean().backward()
        if step == 3:                               # first local step; the sync follows its inner update
            mean_grad = eng.finalize_grads().clone()
            dist.all_reduce(mean_grad)
            mean_grad /= world
        res.optim.step()
        if step == 2:                               # end of the synchronous warm-up
            assert lsgd._baseline_set and torch.equal(lsgd.last_synced, eng.master)
            base = eng.master.clone()
    assert lsgd.outer_steps == 1
    pg = 0.1 * mean_grad                            # base - mean_r(base - 0.1 * g_r)
    expect = base - 0.7 * (pg + 0.9 * pg)           # first outer step: momentum buffer = pg
    assert torch.allclose(eng.master, expect, atol=1e-6), (eng.master - expect).abs().max()


def test_sharded_local_sgd_warmup_baseline_gloo():
    from tests.dist_utils import run_distributed

    run_distributed(_warmup_baseline, world=2)


def _async_mode(rank, world):
    """Asynchronous (wall-clock) synchronisation: the decision comes from the mean of the ranks' clocks and the
    replicas' total step count; the outer state lives on the host between outer steps (``cpu_offload``)."""
    from atorch_b200.local_sgd import LocalSGDConfig, OuterOptimizerConfig, OuterOptimPeriodicModelAverager

    cfg = LocalSGDConfig(use_async=True, local_sgd_sync_time=10.0, min_total_global_steps=6, local_sgd_warmup_steps=1,
                         use_step_weight=True, cpu_offload=True)
    av = OuterOptimPeriodicModelAverager(local_sgd_config=cfg, outer_optim_config=OuterOptimizerConfig(
        torch.optim.SGD, {"lr": 1.0, "momentum": 0.0}))
    now = [1000.0 + 3.0 * rank]            # the ranks' clocks disagree; the mean decides
    av._clock = lambda: now[0]
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.zeros(4))
    synced = []
    for step in range(12):
        with torch.no_grad():
            # the warm-up step is synchronous (same update everywhere); then rank r drifts by r + 1 per step
            p.add_(1.0 if step == 0 else float(rank + 1))
        before = av.outer_steps if av._fused_sgd else None
        s0 = av._step_at_last_sync
        av.average_parameters([p])
        if av._step_at_last_sync != s0 or (step == 1):
            synced.append(step)
        now[0] += 4.0                      # 4 s per step: 10 s are over after 3 steps, 6 total steps after 3 (2 ranks)
        del before
    # warm-up step 0: no sync; step 1: first sync starts the clock; then every third step (12 s >= 10 s, 6 steps)
    assert synced == [1, 4, 7, 10], synced
    # equal step counts -> weights 1/2: after a sync every replica holds the mean of the two drifts
    assert av.last_synced.device.type == "cpu"
    vals = [torch.zeros(4) for _ in range(world)]
    torch.distributed.all_gather(vals, p.detach())
    assert torch.allclose(vals[0] - vals[1], torch.full((4,), -1.0)), vals   # one local step apart since step 10


def test_async_wall_clock_sync_step_weight_and_cpu_offload_gloo():
    run_distributed(_async_mode, world=2)
