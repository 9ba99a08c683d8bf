"""FP8 block-scaled modules on CPU (reference math): quantise/dequantise error, ScaledLinear and the
grouped linear against bf16/fp32 linears, precision switching, module conversion."""
import torch
import torch.nn as nn

from atorch_b200.modules.fp8 import (ATorchGroupedLinear, PrecisionSwitchableLinear, ScaledLinear,
                                     convert_linears_to_fp8, get_fp8_module_count, set_linear_modules_precision)
from atorch_b200.modules.fp8 import quantize as Q


def test_quantize_roundtrip():
    torch.manual_seed(0)
    x = torch.randn(64, 256) * 3
    q, s = Q.tile_quantize_reference(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (64, 2)
    assert (Q.dequantize_reference(q, s, False) - x).abs().max() < 0.07 * x.abs().max()
    qp, sp = Q.tile_quantize_reference(x, pow2=True)
    assert torch.equal(torch.log2(sp), torch.log2(sp).round())
    w = torch.randn(256, 128)
    qb, sb = Q.block_quantize_reference(w)
    assert sb.shape == (2, 1)
    assert (Q.dequantize_reference(qb, sb, True) - w).abs().max() < 0.07 * w.abs().max()


def test_scaled_linear_close_to_dense():
    torch.manual_seed(1)
    lin = nn.Linear(256, 128, bias=True).to(torch.bfloat16)
    sl = ScaledLinear.from_linear(lin)
    x = torch.randn(128, 256, dtype=torch.bfloat16, requires_grad=True)
    y = sl(x)
    ref = nn.functional.linear(x.float(), lin.weight.float(), lin.bias.float())
    assert (y.float() - ref).abs().max() < 0.06 * ref.abs().max()
    y.float().pow(2).sum().backward()
    xr = x.detach().float().requires_grad_()
    wr = lin.weight.detach().float().requires_grad_()
    nn.functional.linear(xr, wr, lin.bias.float()).pow(2).sum().backward()
    assert (x.grad.float() - xr.grad).abs().max() < 0.08 * xr.grad.abs().max()
    assert (lin.weight.grad.float() - wr.grad).abs().max() < 0.08 * wr.grad.abs().max()


def test_switchable_and_conversion():
    model = nn.Sequential(nn.Linear(128, 256), nn.ReLU(), nn.Linear(256, 100))
    n = convert_linears_to_fp8(model, {"precision_switchable": True})
    assert n == 1 and isinstance(model[0], PrecisionSwitchableLinear) and type(model[2]) is nn.Linear
    assert get_fp8_module_count(model) == (1, 0, 1)
    set_linear_modules_precision(model, precision="original")
    assert get_fp8_module_count(model) == (0, 1, 1)
    x = torch.randn(4, 128)
    assert model(x).shape == (4, 100)


def test_grouped_linear():
    torch.manual_seed(2)
    gl = ATorchGroupedLinear(3, 128, 256, fp8=True)
    x = torch.randn(384, 128, dtype=torch.bfloat16, requires_grad=True)
    splits = [128, 0, 256]
    y = gl(x, splits)
    ref = torch.cat([x[:128].float() @ gl.weight0.float().t(), x[128:].float() @ gl.weight2.float().t()])
    assert (y.float() - ref).abs().max() < 0.06 * ref.abs().max()
    y.float().sum().backward()
    assert gl.weight0.grad is not None and gl.weight1.grad.abs().sum() == 0
