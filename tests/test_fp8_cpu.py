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


def test_grouped_linear_weight_cache_and_wgrad_accumulation():
    """ATorchGroupedLinear: later micro-batches reuse the quantised weights of the first one; with
    fuse_wgrad_accumulation the weight gradients of all micro-batches add up in main_grad."""
    import torch

    from atorch_b200.modules.fp8.quantized_grouped_linear import ATorchGroupedLinear

    torch.manual_seed(0)
    lin = ATorchGroupedLinear(2, 128, 256, fp8=True, fuse_wgrad_accumulation=True)
    ref = ATorchGroupedLinear(2, 128, 256, fp8=True)
    for i in range(2):
        getattr(ref, f"weight{i}").data.copy_(getattr(lin, f"weight{i}").data)
        w = getattr(lin, f"weight{i}")
        w.main_grad = torch.zeros_like(w, dtype=torch.float32)
    xs = [torch.randn(256, 128, dtype=torch.bfloat16) for _ in range(3)]
    for mb, x in enumerate(xs):
        lin(x, [128, 128], is_first_microbatch=(mb == 0)).float().sum().backward()
        ref(x, [128, 128]).float().sum().backward()
    assert lin.quant_cache.misses == 2 and lin.quant_cache.hits == 4          # quantised once per weight
    assert ref.quant_cache.misses == 6
    for i in range(2):
        w, wr = getattr(lin, f"weight{i}"), getattr(ref, f"weight{i}")
        assert w.grad is None and getattr(w, "grad_added_to_main_grad", False)
        assert torch.allclose(w.main_grad, wr.grad.float(), rtol=2e-2, atol=2e-1)
    # a changed weight is re-quantised even when the caller says "not the first micro-batch"
    with torch.no_grad():
        lin.weight0.add_(1.0)
    lin(xs[0], [128, 128], is_first_microbatch=False)
    assert lin.quant_cache.misses == 3
