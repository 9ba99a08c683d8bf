"""tcgen05 GEMM against an fp32 PyTorch reference: all operand layouts, ragged shapes, epilogues."""
import pytest
import torch

from atorch_b200 import _lib
from atorch_b200.ops import gemm, gemm_reference, linear

pytestmark = pytest.mark.gpu


def _mk(rows, cols, dev="cuda"):
    return (torch.randn(rows, cols, device=dev, dtype=torch.float32) * 0.5).to(torch.bfloat16)


def _check(out, ref, K):
    torch.cuda.synchronize()
    _lib.check_status(out.device)
    err = (out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err / scale < 2e-2, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (384, 264, 136), (1000, 1032, 520),
                                   (4096, 4096, 1024), (128, 4096, 4096), (72, 96, 40)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(M + N + K)
    a = _mk(K, M) if a_mn else _mk(M, K)
    b = _mk(K, N) if b_mn else _mk(N, K)
    ref = gemm_reference(a, b, a_mn, b_mn, out_dtype=torch.float32)
    for tile_n in (128, 256):
        out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, tile_n=tile_n, kernel="1cta")
        _check(out, ref, K)
    for tile_n in (0, 128, 256):
        out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, kernel="2cta", tile_n=tile_n)
        _check(out, ref, K)


def test_gemm_fp32_out_accumulate_alpha_bias():
    torch.manual_seed(1)
    M, N, K = 512, 768, 384
    a, b = _mk(M, K), _mk(N, K)
    bias = _mk(1, N)[0]
    c0 = torch.randn(M, N, device="cuda")
    out = c0.clone()
    gemm(a, b, out=out, accumulate=True, alpha=0.5, bias=bias)
    ref = c0 + 0.5 * (a.float() @ b.float().t()) + bias.float()
    _check(out, ref, K)
    c1 = _mk(M, N)
    out = c1.clone()
    gemm(a, b, out=out, accumulate=True)
    _check(out, c1.float() + a.float() @ b.float().t(), K)


def test_gemm_strided_operands():
    torch.manual_seed(2)
    big = _mk(512, 1024)
    a = big[:, 256:768]  # pitch 1024, K = 512
    b = _mk(256, 512)
    out = gemm(a, b)
    _check(out, a.float() @ b.float().t(), 512)


def test_gemm_many_tiles_persistent():
    # more tiles than SMs: exercises accumulator double buffering and ring wrap-around
    torch.manual_seed(3)
    M, N, K = 4096, 11008, 512
    a, b = _mk(M, K), _mk(N, K)
    out = gemm(a, b)
    idx = torch.randint(0, M, (64,), device="cuda")
    ref = a[idx].float() @ b.float().t()
    _check(out[idx], ref, K)
    out2 = gemm(a, b, max_ctas=7)
    assert torch.equal(out, out2)
    out3 = gemm(a, b, kernel="1cta")
    _check(out3[idx], ref, K)
    c0 = torch.randn(M, N, device="cuda")
    o4 = c0.clone()
    gemm(a, b, out=o4, accumulate=True, alpha=0.5, kernel="2cta")
    _check(o4[idx], c0[idx] + 0.5 * ref, K)


def test_residual_epilogue():
    torch.manual_seed(6)
    M, N, K = 512, 4096, 256
    a, b, r = _mk(M, K), _mk(N, K), _mk(M, N)
    for kern in ("1cta", "2cta"):
        out = gemm(a, b, residual=r, kernel=kern)
        _check(out, r.float() + a.float() @ b.float().t(), K)


def test_linear_autograd_matches_torch():
    torch.manual_seed(4)
    x = _mk(96, 256).requires_grad_()
    w = _mk(512, 256).requires_grad_()
    res = _mk(96, 512).requires_grad_()
    y = linear(x, w, residual=res)
    dy = _mk(96, 512)
    y.backward(dy)
    xr, wr, rr = (t.detach().float().requires_grad_() for t in (x, w, res))
    yr = rr + xr @ wr.t()
    yr.backward(dy.float())
    _check(y, yr, 256)
    _check(x.grad, xr.grad, 512)
    _check(w.grad, wr.grad, 96)
    assert torch.equal(res.grad, dy)


def test_linear_main_grad_accumulation():
    torch.manual_seed(5)
    x = _mk(128, 256).requires_grad_()
    w = _mk(384, 256).requires_grad_()
    w.main_grad = torch.zeros(384, 256, device="cuda", dtype=torch.float32)
    dy = _mk(128, 384)
    for _ in range(2):
        linear(x, w).backward(dy)
    assert w.grad is None
    ref = 2 * (dy.float().t() @ x.detach().float())
    _check(w.main_grad, ref, 128)


def test_grouped_gemm_with_device_counts():
    """ops.gemm(groups=...): slot groups filled up to device-resident counts (zero beyond), empty tiles
    skipped and written as zeros, one stacked B operand per expert, k-block skipping in the wgrad form."""
    from atorch_b200 import ops

    torch.manual_seed(4)
    E, W, cap, K, N = 2, 3, 512, 256, 384
    G = E * W
    counts = torch.tensor([512, 0, 130, 256, 257, 1], dtype=torch.int32, device="cuda")
    x = torch.randn(G * cap, K, device="cuda", dtype=torch.bfloat16)
    rows = torch.arange(G * cap, device="cuda")
    valid = (rows % cap) < counts[rows // cap]
    x[~valid] = 0
    w = (0.1 * torch.randn(E, N, K, device="cuda")).bfloat16()
    out = torch.full((G * cap, N), 7.0, device="cuda", dtype=torch.bfloat16)      # stale contents everywhere
    ops.gemm(x, w.reshape(E * N, K), out=out, groups={"counts": counts, "m_rows": cap, "n_b": E, "bm_rows": W * cap})
    ref = torch.cat([x[e * W * cap:(e + 1) * W * cap].float() @ w[e].float().t() for e in range(E)])
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    assert (out[~valid] == 0).all()
    # dgrad form: B read MN-major, stacked along its row (k) axis
    dy = torch.randn(G * cap, N, device="cuda", dtype=torch.bfloat16)
    dy[~valid] = 0
    dx = ops.gemm(dy, w.reshape(E * N, K), b_mn=True, groups={"counts": counts, "m_rows": cap, "n_b": E,
                                                                "bm_rows": W * cap})
    ref = torch.cat([dy[e * W * cap:(e + 1) * W * cap].float() @ w[e].float() for e in range(E)])
    assert torch.allclose(dx.float(), ref, rtol=2e-2, atol=3e-2)
    # wgrad form: the reduction runs over the slots, empty k-blocks are skipped
    for e in range(E):
        sl = slice(e * W * cap, (e + 1) * W * cap)
        dw = ops.gemm(dy[sl], x[sl], a_mn=True, b_mn=True, groups={"counts": counts[e * W:(e + 1) * W], "k_rows": cap})
        ref = dy[sl].float().t() @ x[sl].float()
        assert torch.allclose(dw.float(), ref, rtol=2e-2, atol=2e-1), (dw.float() - ref).abs().max()
    # all groups empty: zeros, not stale data
    zc = torch.zeros(W, dtype=torch.int32, device="cuda")
    dw = torch.full((N, K), 3.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm(dy[:W * cap], x[:W * cap], a_mn=True, b_mn=True, out=dw, groups={"counts": zc, "k_rows": cap})
    assert (dw == 0).all()


@pytest.mark.parametrize("T,H,F", [(512, 1024, 1408), (1000, 512, 2752), (4096, 4096, 11008)])
def test_linear_swiglu_epilogue_matches_separate_kernels(T, H, F):
    """SwiGLU in the GEMM epilogue: the activation and the kept gate|up tensor are bit-identical to the GEMM
    followed by the SwiGLU kernel, with and without gradients; gradients agree with the two-op form."""
    from atorch_b200 import ops

    torch.manual_seed(T + F)
    x = _mk(T, H)
    w = (_mk(2 * F, H) * 0.1).to(torch.bfloat16)
    with torch.no_grad():
        ref = ops.swiglu(ops.linear(x, w))
        out = ops.linear_swiglu(x, w)
    torch.cuda.synchronize()
    _lib.check_status(x.device)
    assert torch.equal(out, ref)
    xa, wa = x.clone().requires_grad_(), w.clone().requires_grad_()
    xb, wb = x.clone().requires_grad_(), w.clone().requires_grad_()
    ya = ops.linear_swiglu(xa, wa)
    yb = ops.swiglu(ops.linear(xb, wb))
    assert type(ya.grad_fn).__name__ == "_LinearSwiGLUBackward" and torch.equal(ya, yb)
    dy = _mk(T, F)
    ya.backward(dy)
    yb.backward(dy)
    torch.cuda.synchronize()
    _lib.check_status(x.device)
    assert torch.equal(xa.grad, xb.grad) and torch.equal(wa.grad, wb.grad)
    # against fp32 math
    g = x.float() @ w.float().t()
    full = torch.nn.functional.silu(g[:, :F]) * g[:, F:]
    _check(out, full, H)


def test_dynamic_tile_schedule_matches_static():
    """Tiles handed out by the atomic counter give bit-identical results to the fixed-stride schedule, launch after
    launch (the counters are left at zero), on two streams at once, and while another kernel shares the SMs."""
    L = _lib.lib()
    torch.manual_seed(11)
    side = torch.cuda.Stream()
    try:
        for M, N, K, a_mn, b_mn in [(4096, 4096, 1024, False, False), (4096, 11008, 512, False, True),
                                    (2048 + 72, 4096 + 8, 1024 + 40, True, True), (8192, 8192, 256, False, False)]:
            a = _mk(K, M) if a_mn else _mk(M, K)
            b = _mk(K, N) if b_mn else _mk(N, K)
            L.atb_gemm_set_dynamic(0)
            ref = gemm(a, b, a_mn=a_mn, b_mn=b_mn, kernel="2cta")
            L.atb_gemm_set_dynamic(1)
            outs = [gemm(a, b, a_mn=a_mn, b_mn=b_mn, kernel="2cta") for _ in range(3)]
            filler = torch.empty(64 << 20, device="cuda")
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):                       # a second stream has counters of its own
                for _ in range(4):
                    filler.normal_()
                other = gemm(a, b, a_mn=a_mn, b_mn=b_mn, kernel="2cta")
            busy = gemm(a, b, a_mn=a_mn, b_mn=b_mn, kernel="2cta")
            torch.cuda.synchronize()
            _lib.check_status(ref.device)
            for o in outs + [other, busy]:
                assert torch.equal(o, ref)
    finally:
        L.atb_gemm_set_dynamic(1)
