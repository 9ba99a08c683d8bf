"""AGD, WSAM, BF16Optimizer, AdamL on small CPU problems."""
import math

import torch
import torch.nn as nn

from atorch_b200.optimizers import AGD, AdamL, BF16Optimizer, WeightedSAM


def test_agd_first_steps_follow_the_update_rule():
    p = nn.Parameter(torch.tensor([1.0, -2.0, 3.0]))
    opt = AGD([p], lr=0.1, betas=(0.9, 0.999), delta=1e-5, weight_decay=0.0)
    g1 = torch.tensor([0.5, -1.0, 2.0])
    p.grad = g1.clone()
    opt.step()
    m = 0.1 * g1
    s = m / 0.1
    v = 0.001 * s * s
    den = torch.maximum(v.sqrt(), torch.full_like(v, 1e-5 * math.sqrt(0.001)))
    expect = torch.tensor([1.0, -2.0, 3.0]) - 0.1 * math.sqrt(0.001) / 0.1 * (m / den)
    assert torch.allclose(p.detach(), expect, atol=1e-6)
    g2 = torch.tensor([0.4, -1.1, 1.0])
    p.grad = g2.clone()
    opt.step()
    m2 = 0.9 * m + 0.1 * g2
    s2 = m2 / (1 - 0.81) - m / 0.1
    v2 = 0.999 * v + 0.001 * s2 * s2
    den2 = torch.maximum(v2.sqrt(), torch.full_like(v2, 1e-5 * math.sqrt(1 - 0.999 ** 2)))
    expect2 = expect - 0.1 * math.sqrt(1 - 0.999 ** 2) / (1 - 0.81) * (m2 / den2)
    assert torch.allclose(p.detach(), expect2, atol=1e-6)


def test_agd_converges_and_variants_run():
    torch.manual_seed(0)
    for kw in ({}, {"amsgrad": True}, {"win": True}, {"clip": 1.0}, {"weight_decouple": False, "weight_decay": 0.01}):
        w = nn.Parameter(torch.randn(10))
        target = torch.arange(10.0)
        opt = AGD([w], lr=0.05, **kw)
        first = None
        for _ in range(300):
            opt.zero_grad()
            loss = ((w - target) ** 2).sum()
            first = first if first is not None else loss.item()
            loss.backward()
            opt.step()
        assert loss.item() < first * (0.5 if "clip" in kw else 0.05), kw


def test_wsam_decoupled_matches_manual():
    torch.manual_seed(1)
    model = nn.Linear(4, 1, bias=False)
    base = torch.optim.SGD(model.parameters(), lr=0.1)
    opt = WeightedSAM(model, base, rho=0.05, gamma=0.5, decouple=True)
    x, y = torch.randn(8, 4), torch.randn(8, 1)
    w0 = model.weight.detach().clone()

    def closure():
        opt.zero_grad()
        loss = ((model(x) - y) ** 2).mean()
        loss.backward()
        return loss
    opt.step(closure)

    def grad_at(w):
        w = w.clone().requires_grad_()
        ((x @ w.t() - y) ** 2).mean().backward()
        return w.grad
    g = grad_at(w0)
    e = 0.05 * g / (g.norm() + 1e-12)
    gs = grad_at(w0 + e)
    expect = w0 - 0.1 * g - 0.1 * 1.0 * (gs - g)
    assert torch.allclose(model.weight.detach(), expect, atol=1e-6)


def test_bf16_optimizer_keeps_fp32_master():
    torch.manual_seed(2)
    model = nn.Linear(16, 16).to(torch.bfloat16)
    opt = BF16Optimizer(torch.optim.SGD(model.parameters(), lr=1e-3))
    ref = [p.detach().float().clone() for p in model.parameters()]
    for _ in range(50):
        opt.zero_grad()
        for p in model.parameters():
            p.grad = torch.full_like(p, 0.01)
        opt.step()
    # 50 steps of 1e-5 each would be lost entirely in pure bf16 arithmetic for weights near 0.1
    for p, r in zip(model.parameters(), ref):
        assert torch.allclose(p.float(), (r - 50 * 1e-3 * 0.01).bfloat16().float(), atol=1e-2)
    sd = opt.state_dict()
    assert "fp32_from_fp16" in sd and "optimizer_state_dict" in sd
    opt.load_state_dict(sd)


def test_adaml_l1_zeroes_small_weights():
    p = nn.Parameter(torch.tensor([0.0005, -0.5, 0.3]))
    opt = AdamL([p], lr=0.01, l1=0.2)
    p.grad = torch.zeros(3)
    opt.step()
    assert p[0].item() == 0.0 and abs(p[1].item() + 0.498) < 1e-6


def test_partition_adam_matches_adamw_and_keeps_state_in_host_blocks():
    import torch.nn as nn

    from atorch_b200.optimizers import PartitionAdam

    torch.manual_seed(0)
    a = nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 4))
    b = nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 4))
    b.load_state_dict(a.state_dict())
    groups = lambda m: [{"params": list(m[0].parameters())}, {"params": list(m[2].parameters()), "lr": 3e-3}]  # noqa: E731
    oa = PartitionAdam(groups(a), lr=1e-3, weight_decay=0.01)
    ob = torch.optim.AdamW(groups(b), lr=1e-3, weight_decay=0.01)
    for i in range(5):
        x = torch.randn(8, 16, generator=torch.Generator().manual_seed(i))
        for m, o in ((a, oa), (b, ob)):
            o.zero_grad()
            m(x).pow(2).mean().backward()
            o.step()
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.allclose(p, q, atol=1e-6), (p - q).abs().max()
    blk = oa.state["group0"]["state_block"]
    assert blk.numel() == 2 * (16 * 32 + 32) and blk.abs().sum() > 0 and oa.param_groups[1]["step"] == 5


def test_mup_qkv_and_q_layers_zero_the_query_rows():
    import torch.nn as nn

    from atorch_b200.mup import MupModule, QKVLayer, QLayer, set_base_shapes

    class Attn(MupModule):
        def __init__(self):
            super().__init__()
            self.qkv, self.q, self.plain = QKVLayer(8, 24), QLayer(8, 8), QKVLayer(8, 24, q_zero_init=False)

    m = Attn()
    set_base_shapes(m, None)
    m.mup_initial("mup")
    assert m.qkv.weight[:8].abs().sum() == 0 and m.qkv.weight[8:].abs().sum() > 0
    assert m.q.weight.abs().sum() == 0 and m.plain.weight[:8].abs().sum() > 0
    del nn
