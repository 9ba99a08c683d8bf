"""FP8 quantisers and the block-scaled tcgen05 GEMM against the PyTorch reference math."""
import pytest
import torch

from atorch_b200 import _lib
from atorch_b200.modules.fp8 import ScaledLinear
from atorch_b200.modules.fp8 import quantize as Q

pytestmark = pytest.mark.gpu


def _x(r, c, scale=2.0):
    return (torch.randn(r, c, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("pow2", [False, True])
def test_quantisers_match_reference(pow2):
    torch.manual_seed(0)
    x = _x(384, 512)
    q, s = Q.tile_quantize(x, pow2)
    qr, sr = Q.tile_quantize_reference(x, pow2)
    assert torch.allclose(s, sr, rtol=1e-6)
    assert (q.float() - qr.float()).abs().max() <= 32      # at most one e4m3 step near a rounding tie
    assert (q.view(torch.uint8) != qr.view(torch.uint8)).float().mean() < 1e-2
    qt, st = Q.tile_quantize_transposed(x, pow2)
    qtr, str_ = Q.tile_quantize_reference(x.t().contiguous(), pow2)
    assert qt.shape == (512, 384) and torch.allclose(st, str_, rtol=1e-6)
    assert (qt.view(torch.uint8) != qtr.view(torch.uint8)).float().mean() < 1e-2
    w = _x(256, 384, 0.05)
    qb, sb, qbt = Q.block_quantize(w, with_transpose=True, pow2=pow2)
    qbr, sbr = Q.block_quantize_reference(w, pow2)
    assert torch.allclose(sb, sbr, rtol=1e-6)
    assert (qb.view(torch.uint8) != qbr.view(torch.uint8)).float().mean() < 1e-2
    assert torch.equal(qbt.view(torch.uint8), qb.view(torch.uint8).t().contiguous())
    d = Q.dequantize(qb, sb, True)
    assert torch.allclose(d.float(), Q.dequantize_reference(qbr, sbr, True), rtol=2e-2, atol=1e-3)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1000, 256, 1024), (4096, 1024, 4096)])
def test_scaled_gemm(M, N, K):
    torch.manual_seed(M + N)
    a, b = _x(M, K, 1.0), _x(N, K, 0.1)
    aq, a_s = Q.tile_quantize(a)
    bq, b_s = Q.block_quantize(b)
    out = Q.scaled_gemm(aq, a_s, bq, b_s)
    torch.cuda.synchronize()
    _lib.check_status(a.device)
    ref = Q.scaled_gemm_reference(aq, a_s, bq, b_s, False, torch.float32)
    assert (out.float() - ref).abs().max() < 2e-2 * ref.abs().max()
    dense = a.float() @ b.float().t()
    assert (out.float() - dense).abs().max() < 8e-2 * dense.abs().max()
    bq2, b_s2 = Q.tile_quantize(b)                       # per-row scales on B
    acc = torch.randn(M, N, device="cuda")
    o2 = acc.clone()
    Q.scaled_gemm(aq, a_s, bq2, b_s2, b_row_mode=True, out=o2, accumulate=True)
    ref2 = Q.scaled_gemm_reference(aq, a_s, bq2, b_s2, True, torch.float32) + acc
    assert (o2 - ref2).abs().max() < 2e-2 * ref2.abs().max()


def test_scaled_linear_training_step():
    torch.manual_seed(3)
    lin = torch.nn.Linear(512, 256, bias=False, device="cuda", dtype=torch.bfloat16)
    sl = ScaledLinear.from_linear(lin)
    x = _x(256, 512, 1.0).requires_grad_()
    y = sl(x)
    dy = _x(256, 256, 1.0)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), lin.weight.detach().float().requires_grad_()
    (xr @ wr.t()).backward(dy.float())
    for got, ref in ((y, xr @ wr.t()), (x.grad, xr.grad), (lin.weight.grad, wr.grad)):
        assert (got.float() - ref).abs().max() < 8e-2 * ref.abs().max()
