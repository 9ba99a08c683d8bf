"""Integer group quantisation and optimizer-state packing kernels against their PyTorch references."""
import pytest
import torch

from atorch_b200.ops import lowbit, quantizer

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quantize_dequantize(bits, sym, dtype):
    torch.manual_seed(0)
    x = torch.randn(64 * 2048, device="cuda").to(dtype)
    q, p = quantizer.quantize(x, 64, bits, sym)
    qr, pr = quantizer.quantize_reference(x, 64, bits, sym)
    assert torch.allclose(p, pr.to(p.device), rtol=1e-5, atol=1e-7)
    assert (q != qr).float().mean() < 2e-3
    d = quantizer.dequantize(q, p, 64, bits, sym, torch.float32)
    dr = quantizer.dequantize_reference(q, p, 64, bits, sym, torch.float32)
    assert torch.allclose(d, dr, rtol=1e-5, atol=1e-6)
    assert (d - x.float()).abs().max() < (0.03 if bits == 8 else 0.5)


def test_swizzle_and_reduce():
    torch.manual_seed(1)
    x = torch.randn(32 * 256, device="cuda", dtype=torch.bfloat16)
    q, p = quantizer.swizzle_quant(x, 32, 8, True, 2, 2, 4)
    gm = quantizer.swizzle_group_map(32, 2, 2, 4, "cuda").long()
    q0, p0 = quantizer.quantize(x, 32, 8, True)
    assert torch.equal(q.view(32, -1)[gm], q0.view(32, -1)) and torch.equal(p[gm], p0)
    parts = [torch.randn(8 * 512, device="cuda", dtype=torch.bfloat16) for _ in range(8)]
    qs, ps = zip(*(quantizer.quantize(t, 8, 8, True) for t in parts))
    qo, po = quantizer.quantized_reduction(torch.cat(qs), torch.cat(ps), 64, 8, 8, True, 8)
    got = quantizer.dequantize(qo, po, 8, 8, True, torch.float32)
    ref = sum(quantizer.dequantize(a, b, 8, 8, True, torch.float32) for a, b in zip(qs, ps))
    assert (got - ref).abs().max() < 0.05 * ref.abs().max()


def test_state_packing():
    torch.manual_seed(2)
    x = torch.randn(100000, device="cuda")
    for bits in (8, 16):
        c, am = lowbit.pack_absmax_linear(x, bits, 2048)
        back = lowbit.unpack_absmax_linear(c, am, bits, 2048)
        assert (back - x).abs().max() < (0.03 if bits == 8 else 2e-4)
    for bits, gs in ((4, 128), (8, 2048)):
        qm = lowbit.create_dynamic_map(True, bits).cuda()
        c, am = lowbit.pack_nonlinear(x, qm, bits, gs)
        back = lowbit.unpack_nonlinear(c, am, qm, x.numel(), bits, gs)
        cpu_c, cpu_am = lowbit.pack_nonlinear(x.cpu(), qm.cpu(), bits, gs)
        ref = lowbit.unpack_nonlinear(cpu_c, cpu_am, qm.cpu(), x.numel(), bits, gs)
        assert (back.cpu() - ref).abs().max() < 1e-5
        s1, _ = lowbit.pack_nonlinear(x, qm, bits, gs, stochastic=True, seed=1)
        s2, _ = lowbit.pack_nonlinear(x, qm, bits, gs, stochastic=True, seed=1)
        s3, _ = lowbit.pack_nonlinear(x, qm, bits, gs, stochastic=True, seed=7)
        assert torch.equal(s1, s2) and not torch.equal(s1, s3)
        mean_err = (lowbit.unpack_nonlinear(s1, am, qm, x.numel(), bits, gs) - x).mean().abs()
        assert mean_err < 5e-3            # stochastic rounding is unbiased
