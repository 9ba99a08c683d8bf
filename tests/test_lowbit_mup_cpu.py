"""Quantiser ops, low-bit optimizers and muP on CPU (reference paths)."""
import torch
import torch.nn as nn

from atorch_b200.mup import MuAdam, MuSGD, MupLinear, OutputLayer, set_base_shapes
from atorch_b200.ops import lowbit, quantizer
from atorch_b200.optimizers.low_bit import Q_Adafactor, Q_AdamW, Q_AGD, Q_CAME


def test_group_quantiser_roundtrip_and_reduction():
    torch.manual_seed(0)
    x = torch.randn(8 * 512)
    for bits, tol in ((8, 0.02), (4, 0.35)):
        for sym in (True, False):
            q, p = quantizer.quantize(x, 8, bits, sym)
            assert q.numel() == x.numel() // (2 if bits == 4 else 1) and p.shape == (8, 1 if sym else 2)
            assert (quantizer.dequantize(q, p, 8, bits, sym, torch.float32) - x).abs().max() < tol
    parts = [torch.randn(4 * 256) for _ in range(4)]
    qs, ps = zip(*(quantizer.quantize(t, 4, 8, True) for t in parts))
    qo, po = quantizer.quantized_reduction(torch.cat(qs), torch.cat(ps), 16, 4, 8, True, 4)
    total = quantizer.dequantize(qo, po, 4, 8, True, torch.float32)
    assert (total - sum(parts)).abs().max() < 0.15
    gm = quantizer.swizzle_group_map(16, pipeline_size=2, nodes=2, devices_per_node=2)
    assert sorted(gm.tolist()) == list(range(16))
    q, p = quantizer.swizzle_quant(torch.arange(16 * 4, dtype=torch.float32), 16, 8, True, 2, 2, 2)
    d = quantizer.dequantize(q, p, 16, 8, True, torch.float32).view(16, 4)
    # input group (node 0, dev 1, pipe 0, rest 0) = index 4 lands at (pipe 0, dev 1, node 0) = slot 2... check a permutation
    assert torch.allclose(d.sum(), torch.arange(64.).sum(), rtol=1e-2)


def test_state_codes():
    x = torch.randn(5000)
    c, am = lowbit.pack_absmax_linear(x, 16, 2048)
    assert (lowbit.unpack_absmax_linear(c, am, 16, 2048) - x).abs().max() < 1e-3
    qm = lowbit.create_dynamic_map(True, 8)
    c, am = lowbit.pack_nonlinear(x, qm, 8, 2048)
    assert (lowbit.unpack_nonlinear(c, am, qm, 5000, 8, 2048) - x).abs().max() < 0.1
    c1, _ = lowbit.pack_nonlinear(x, qm, 8, 2048, stochastic=True, seed=1)
    c2, _ = lowbit.pack_nonlinear(x, qm, 8, 2048, stochastic=True, seed=2)
    assert not torch.equal(c1, c2)


def test_lowbit_optimizers_converge():
    for cls, kw in ((Q_AdamW, dict(lr=0.05, weight_decay=0.0)), (Q_AGD, dict(lr=0.05)),
                    (Q_Adafactor, dict(lr=0.05)), (Q_CAME, dict(lr=0.02))):
        torch.manual_seed(1)
        w = nn.Parameter(torch.randn(80, 64))           # 5120 elements: quantised states
        target = torch.randn(80, 64)
        opt = cls([w], q_bits=8, **kw)
        first = None
        for _ in range(150):
            opt.zero_grad()
            loss = ((w - target) ** 2).mean()
            first = first if first is not None else loss.item()
            loss.backward()
            opt.step()
        assert loss.item() < 0.3 * first, (cls.__name__, first, loss.item())


def test_mup_scaling():
    def make(width):
        return nn.Sequential(MupLinear(8, width), nn.ReLU(), MupLinear(width, width), nn.ReLU(), OutputLayer(width, 4, weight_zero_init=True))
    base, delta, model = make(16), make(32), make(64)
    set_base_shapes(model, base, delta)
    assert model[2].weight.infshape.ninf() == 2 and model[2].weight.infshape.width_mult() == 4.0
    assert model[0].weight.infshape.ninf() == 1 and model[4].width_mult() == 4.0
    for m in model:
        if hasattr(m, "mup_initial"):
            m.mup_initial()
    assert model[4].weight.abs().sum() == 0
    opt = MuAdam(model.parameters(), lr=1e-2)
    lrs = sorted({g["lr"] for g in opt.param_groups})
    assert lrs == [1e-2 / 4, 1e-2] and isinstance(opt, torch.optim.AdamW)
    opt2 = MuSGD(model.parameters(), lr=1e-1)
    assert any(abs(g["lr"] - 0.4) < 1e-9 for g in opt2.param_groups)
    model(torch.randn(2, 8)).sum().backward()
    opt.step()
