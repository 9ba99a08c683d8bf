"""Row / elementwise sm_100a kernels against fp32 PyTorch references."""
import pytest
import torch

from atorch_b200 import ops

pytestmark = pytest.mark.gpu


def _close(a, b, rtol=2e-2, atol=2e-2):
    torch.cuda.synchronize()
    assert torch.allclose(a.float(), b.float(), rtol=rtol, atol=atol), (a.float() - b.float()).abs().max().item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,N", [(1, 64), (37, 1000), (513, 4096), (64, 8192)])
def test_rmsnorm_fwd_bwd(M, N, dtype):
    torch.manual_seed(0)
    x = torch.randn(M, N, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(N, device="cuda")).to(dtype).requires_grad_()
    dy = torch.randn(M, N, device="cuda", dtype=dtype)
    y = ops.rms_norm(x, w, 1e-5)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(dy.float())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    _close(y, yr, tol, tol)
    _close(x.grad, xr.grad, tol, tol)
    _close(w.grad, wr.grad, tol, tol * max(1.0, M ** 0.5))


def test_rmsnorm_residual_and_main_grad():
    torch.manual_seed(1)
    M, N = 200, 2048
    x = torch.randn(M, N, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(M, N, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(N, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w.main_grad = torch.zeros(N, device="cuda", dtype=torch.float32)
    y, s = ops.rms_norm(x, w, 1e-5, residual=r)
    (y.float().sum() + 2 * s.float().sum()).backward()
    xr = (x.detach().float() + r.detach().float()).to(torch.bfloat16).float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    (yr.sum() + 2 * xr.sum()).backward()
    _close(s, xr)
    _close(y, yr)
    _close(x.grad, xr.grad, 3e-2, 3e-2)
    assert torch.equal(x.grad, r.grad)
    assert w.grad is None
    _close(w.main_grad, wr.grad, 3e-2, 0.5)


@pytest.mark.parametrize("M,N", [(33, 768), (128, 1024)])
def test_layernorm_fwd_bwd(M, N):
    torch.manual_seed(2)
    x = torch.randn(M, N, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(N, device="cuda")).bfloat16().requires_grad_()
    b = (0.1 * torch.randn(N, device="cuda")).bfloat16().requires_grad_()
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    y = ops.layer_norm(x, w, b, 1e-5)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (N,), wr, br, 1e-5)
    yr.backward(dy.float())
    _close(y, yr, 3e-2, 3e-2)
    _close(x.grad, xr.grad, 3e-2, 3e-2)
    _close(w.grad, wr.grad, 3e-2, 0.3)
    _close(b.grad, br.grad, 3e-2, 0.3)


def test_rope_matches_reference_and_is_orthogonal():
    torch.manual_seed(3)
    B, S, nq, nkv, d = 2, 128, 4, 2, 128
    W = (nq + 2 * nkv) * d
    x = torch.randn(B, S, W, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cos, sin = ops.rope_tables(S, d, device="cuda")
    y = ops.rope(x, cos, sin, nq + nkv, d)
    ref = ops.rope_reference(x.detach(), cos, sin, nq + nkv, d)
    _close(y, ref, 1e-2, 1e-2)
    assert torch.equal(y[..., (nq + nkv) * d:], x[..., (nq + nkv) * d:])
    dy = torch.randn_like(y)
    y.backward(dy)
    refg = ops.rope_reference(dy, cos, sin, nq + nkv, d, backward=True)
    _close(x.grad, refg, 1e-2, 1e-2)
    pos = torch.randint(0, S, (B * S,), device="cuda", dtype=torch.int32)
    y2 = ops.rope(x.detach(), cos, sin, nq, d, positions=pos)
    _close(y2, ops.rope_reference(x.detach(), cos, sin, nq, d, positions=pos), 1e-2, 1e-2)


def test_rope_in_place_matches_out_of_place():
    torch.manual_seed(5)
    B, S, nq, nkv, d = 2, 128, 4, 4, 128
    W = (nq + 2 * nkv) * d
    x = torch.randn(B, S, W, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cos, sin = ops.rope_tables(S, d, device="cuda")
    ref = ops.rope(x, cos, sin, nq + nkv, d)
    dy = torch.randn_like(ref)
    ref.backward(dy.clone())
    g_ref, x.grad = x.grad.clone(), None
    h = x * 1.0                                  # a non-leaf that nothing else reads
    y = ops.rope(h, cos, sin, nq + nkv, d, inplace=True)
    assert y.data_ptr() == h.data_ptr()          # rotated where it is
    assert torch.equal(y, ref)
    y.backward(dy.clone())
    assert torch.equal(x.grad, g_ref)
    # a leaf is never overwritten
    z = ops.rope(x, cos, sin, nq + nkv, d, inplace=True)
    assert z.data_ptr() != x.data_ptr()


def test_swiglu_fwd_bwd():
    torch.manual_seed(4)
    gu = torch.randn(300, 2 * 1376, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(300, 1376, device="cuda", dtype=torch.bfloat16)
    y = ops.swiglu(gu)
    y.backward(dy)
    gr = gu.detach().float().requires_grad_()
    yr = torch.nn.functional.silu(gr[:, :1376]) * gr[:, 1376:]
    yr.backward(dy.float())
    _close(y, yr)
    _close(gu.grad, gr.grad, 3e-2, 3e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("V", [32000, 1003])
@pytest.mark.parametrize("smooth,z", [(0.0, 0.0), (0.1, 1e-4)])
def test_cross_entropy(V, dtype, smooth, z):
    torch.manual_seed(5)
    rows = 257
    Vp = (V + 7) // 8 * 8
    buf = torch.randn(rows, Vp, device="cuda", dtype=dtype) * 2
    logits = buf[:, :V].detach().requires_grad_()
    labels = torch.randint(0, V, (rows,), device="cuda")
    labels[::7] = -100
    loss = ops.cross_entropy(logits, labels, label_smoothing=smooth, lse_square_scale=z)
    w = torch.rand(rows, device="cuda")
    (loss * w).sum().backward()
    lr = logits.detach().float().requires_grad_()
    ref = ops.cross_entropy_reference(lr, labels, -100, smooth, z)
    (ref * w).sum().backward()
    _close(loss, ref, 1e-3, 1e-3)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    _close(logits.grad, lr.grad, tol, tol)


def test_adamw_and_agd_steps():
    torch.manual_seed(6)
    n = 100003
    for gd in (torch.bfloat16, torch.float32):
        master = torch.randn(n, device="cuda")
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        mr, m2, v2 = master.clone(), m.clone(), v.clone()
        for step in range(1, 4):
            g = torch.randn(n, device="cuda").to(gd)
            ops.adamw_step(master, m, v, g, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=0.5)
            ops.adamw_reference(mr, m2, v2, g, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=0.5)
        _close(master, mr, 1e-5, 1e-5)
        _close(lp, mr.bfloat16(), 1e-2, 1e-2)
        master = torch.randn(n, device="cuda")
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        mr, m2, v2 = master.clone(), m.clone(), v.clone()
        for step in range(1, 4):
            g = torch.randn(n, device="cuda").to(gd)
            ops.agd_step(master, m, v, g, lp, 1e-2, 0.9, 0.999, 1e-5, 0.1, step)
            ops.agd_reference(mr, m2, v2, g, None, 1e-2, 0.9, 0.999, 1e-5, 0.1, step)
        _close(master, mr, 1e-4, 1e-4)


def test_sum_squares_and_outer_sgd():
    torch.manual_seed(7)
    x = torch.randn(1 << 20, device="cuda")
    ref = x.double().pow(2).sum().item()
    assert abs(ops.sum_squares(x).item() - ref) < 2e-6 * ref
    n = 5000
    synced, buf, pg = torch.randn(n, device="cuda"), torch.zeros(n, device="cuda"), torch.randn(n, device="cuda")
    p = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    s2, b2 = synced.clone(), buf.clone()
    for i in range(3):
        ops.outer_sgd_step(synced, buf, pg, p, 0.7, 0.9, True, i == 0)
        ops.outer_sgd_reference(s2, b2, pg, None, 0.7, 0.9, True, i == 0)
    _close(synced, s2, 1e-5, 1e-5)
    _close(p, s2.bfloat16(), 1e-2, 1e-2)


def test_bias_gather_add():
    torch.manual_seed(8)
    inp = torch.randn(100, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    bias = torch.randn(8, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    idx = torch.randint(0, 8, (100,), device="cuda")
    out = ops.bias_gather_add(inp, bias, idx)
    _close(out, ops.bias_gather_add_reference(inp.detach(), bias.detach(), idx))
    out.sum().backward()
    cnt = torch.bincount(idx, minlength=8).float()
    _close(bias.grad, cnt[:, None].expand(8, 256), 1e-2, 1e-2)


def test_rmsnorm_carry_adds_the_residual_gradient_in_the_kernel():
    """``carry=True`` hands x back for the residual path: no copy, and the gradient through it is added inside the
    backward kernel. Same numbers as the plain form plus autograd's own add."""
    torch.manual_seed(8)
    x = torch.randn(512, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(4096, device="cuda", dtype=torch.bfloat16)
    dy, dres = torch.randn_like(x), torch.randn_like(x)
    xa, wa = x.clone().requires_grad_(), w.clone().requires_grad_()
    h = xa * 1.0
    y, carried = ops.rms_norm(h, wa, 1e-5, carry=True)
    assert carried.data_ptr() == h.data_ptr() and torch.equal(carried, h)
    torch.autograd.backward([y, carried], [dy, dres])
    xb, wb = x.clone().requires_grad_(), w.clone().requires_grad_()
    y2 = ops.rms_norm(xb, wb, 1e-5)
    assert torch.equal(y, y2)
    y2.backward(dy)
    ref = xb.grad.float() + dres.float()
    _close(xa.grad, ref, 2e-2, 2e-2)
    assert torch.equal(wa.grad, wb.grad)
