"""MoE on CPU: permutation round trip, routers, Grouped_GEMM_MoE against a dense per-token evaluation,
expert parallel (gloo, world 2) against the single-process result for both dispatchers."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from atorch_b200.modules.moe import Experts, Grouped_GEMM_MoE, MOELayer, SwitchGate, TopkGate, TopNRouter
from atorch_b200.ops import moe as moe_ops
from tests.dist_utils import run_distributed


def test_permute_unpermute_roundtrip():
    torch.manual_seed(0)
    x = torch.randn(10, 6)
    idx = torch.randint(0, 4, (10, 2))
    probs = torch.rand(10, 2)
    p, s = moe_ops.permute(x, idx)
    flat = idx.reshape(-1)
    assert torch.equal(flat[s], flat.sort(stable=True).values)
    y = moe_ops.unpermute(p, s, probs, 2, 10)
    assert torch.allclose(y, x * probs.sum(1, keepdim=True), atol=1e-6)
    assert moe_ops.tokens_per_expert(idx, 4).sum() == 20


def _dense_moe(moe, x, w, idx):
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(idx.shape[1]):
            e = idx[t, j].item()
            h = x[t] @ moe.w1[e].t()
            f = moe.expert_intermediate_size
            h = F.silu(h[:f]) * h[f:]
            out[t] += w[t, j] * (h @ moe.w2[e])
    return out


def test_grouped_gemm_moe_matches_dense():
    torch.manual_seed(1)
    moe = Grouped_GEMM_MoE(16, 24, 0.0, num_experts=4, topk=2, use_swiglu=True)
    router = TopNRouter(16, 4, 2, aux_loss_coef=0.01, z_loss_coef=0.001)
    x = torch.randn(12, 16, requires_grad=True)
    w, idx = router(x)
    y = moe(x, w, idx)
    ref = _dense_moe(moe, x, w, idx)
    assert torch.allclose(y, ref, atol=1e-5)
    (y.sum() + router.aux_loss + router.z_loss).backward()
    assert moe.w1.grad is not None and x.grad is not None and router.classifier.weight.grad is not None


def test_capacity_gates():
    torch.manual_seed(2)
    g = TopkGate(8, 4, k=2, capacity_factor=1.0, min_capacity=1)
    l_aux, combine, mask, counts = g(torch.randn(16, 8))
    T, E, C = combine.shape
    assert (T, E) == (16, 4) and C == 8 and mask.sum((0, 2)).max() <= C
    assert (mask.sum((1, 2)) <= 2).all() and l_aux.item() > 0
    kept = mask.any(2).sum(1) > 0
    assert torch.allclose(combine.sum((1, 2))[kept], torch.ones(int(kept.sum())), atol=1e-5)
    s = SwitchGate(8, 4, capacity_factor=1.0, min_capacity=1)
    _, c1, m1, _ = s(torch.randn(16, 8))
    assert (m1.sum((1, 2)) <= 1).all()
    layer = MOELayer(g, Experts(nn.Linear(8, 8), 4))
    y = layer(torch.randn(2, 8, 8))
    assert y.shape == (2, 8, 8)


def _ep(rank, world, dispatcher, out_file):
    from atorch_b200.distributed import distributed as D

    D.create_parallel_group(([("expert", world)], None))
    torch.manual_seed(3)
    full = Grouped_GEMM_MoE(16, 24, 0.0, num_experts=4, topk=2, use_swiglu=True)
    moe = Grouped_GEMM_MoE(16, 24, 0.0, num_experts=4, topk=2, use_swiglu=True, use_expert_parallelism=True,
                           token_dispatcher_type=dispatcher)
    E = moe.num_local_experts
    with torch.no_grad():
        moe.w1.copy_(full.w1[rank * E:(rank + 1) * E])
        moe.w2.copy_(full.w2[rank * E:(rank + 1) * E])
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(6, 16, generator=g, requires_grad=True)
    logits = torch.randn(6, 4, generator=g)
    w, idx = torch.softmax(logits, -1).topk(2, -1)
    y = moe(x, w, idx)
    ref = _dense_moe(full, x.detach(), w, idx)
    assert torch.allclose(y, ref, atol=1e-5), (dispatcher, (y - ref).abs().max())
    y.sum().backward()
    assert x.grad is not None and moe.w1.grad is not None


def test_expert_parallel_gloo(tmp_path):
    for disp in ("AllToAll", "AllGather"):
        run_distributed(_ep, world=2, args=(disp, str(tmp_path / disp)))


def _moe_ddp(rank, world):
    """Dense parameters are averaged over all ranks, expert parameters only over the ranks holding the same
    experts (here: ranks {0, 2} and {1, 3})."""
    import torch.distributed as dist

    from atorch_b200.modules.moe import (Experts, MoEMixtureDistributedDataParallel, set_experts_ddp_process_group)

    groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
    set_experts_ddp_process_group(groups[rank % 2])
    torch.manual_seed(0)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.dense = nn.Linear(4, 4)
            self.experts = Experts(nn.Linear(4, 4), 1)

        def forward(self, x):
            return self.experts(self.dense(x).unsqueeze(0)).squeeze(0) if False else self.dense(x) + \
                self.experts.experts[0](x)
    net = Net()
    with torch.no_grad():                      # ranks of different expert groups hold different experts
        for p in net.experts.parameters():
            p.add_(float(rank % 2))
    m = MoEMixtureDistributedDataParallel(net)
    assert m.moe_params_names == {"experts.experts.0.weight", "experts.experts.0.bias"}
    x = torch.full((2, 4), float(rank + 1))
    m(x).sum().backward()
    gd = net.dense.weight.grad.clone()
    ge = net.experts.experts[0].weight.grad.clone()
    # d/dW of sum(Wx+b) = column sums of x broadcast over rows: 2 * (rank + 1) per entry on this rank
    assert torch.allclose(gd, torch.full_like(gd, 2 * (1 + 2 + 3 + 4) / 4.0))
    mates = [1, 3] if rank % 2 == 0 else [2, 4]
    assert torch.allclose(ge, torch.full_like(ge, 2 * sum(mates) / 2.0)), (rank, ge)


def test_moe_mixture_ddp_gloo():
    run_distributed(_moe_ddp, world=4)


def _group_aware_norms(rank, world):
    import math

    from atorch_b200.distributed.distributed import create_parallel_group, parallel_group
    from atorch_b200.utils.moe_util import clip_grad_norm_, compute_grad_norm_, compute_param_norm_, compute_single_param_std_

    create_parallel_group(([("expert", world)], None))
    torch.manual_seed(1)
    dense = torch.nn.Parameter(torch.randn(5, 3))                  # the same on every rank
    torch.manual_seed(10 + rank)
    expert = torch.nn.Parameter(torch.randn(4, 2))                 # a different expert on every rank
    expert.expert = True
    tagged = torch.nn.Parameter(torch.randn(3))                    # explicit group
    tagged.norm_group = parallel_group("expert")
    for p in (dense, expert, tagged):
        p.grad = p.detach() * 0.5 + 1.0
    params = [dense, expert, tagged]
    everything = [dense.grad.reshape(-1)]
    for r in range(world):
        torch.manual_seed(10 + r)
        e = torch.randn(4, 2)
        t = torch.randn(3)
        everything += [(e * 0.5 + 1.0).reshape(-1), (t * 0.5 + 1.0).reshape(-1)]
    flat = torch.cat(everything)
    for nt in (2.0, 1.0, math.inf):
        got = compute_grad_norm_(params, nt)
        assert torch.allclose(got, torch.linalg.vector_norm(flat, nt), rtol=1e-5), (nt, got)
    assert compute_param_norm_(params).item() > 0
    assert torch.allclose(compute_single_param_std_(dense), dense.detach().std(), rtol=1e-5)
    before = [p.grad.clone() for p in params]
    total = clip_grad_norm_(params, max_norm=1.0)
    coef = 1.0 / (torch.linalg.vector_norm(flat, 2.0) + 1e-6)
    assert torch.allclose(total, torch.linalg.vector_norm(flat, 2.0), rtol=1e-5)
    for p, b in zip(params, before):
        assert torch.allclose(p.grad, b * coef, rtol=1e-5)


def test_norms_over_parameters_partitioned_on_different_groups_gloo():
    from tests.dist_utils import run_distributed

    run_distributed(_group_aware_norms, world=2)
