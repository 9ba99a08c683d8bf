"""The allocation-free RMSNorm backward (`atb_rmsnorm_bwd_noalloc`, csrc/no_alloc.h).

It exists for callers that may not allocate device memory around a kernel call: a host runtime
that owns the whole device arena and only lends out input/output buffers, or a path that must stay
clear of cudaMalloc/cudaFree. The test calls the exported C symbol directly through ctypes, twice
in a row on different data (the built-in scratch keeps the first call's contents, which must not
leak into the second), and compares with the regular entry points (`atb_norm_bwd` + `atb_colsum`),
which get their scratch from the caller. It also checks that oversize problems are refused.

This file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _raw_lib():
    from atorch_b200 import _lib

    assert _lib.lib() is not None
    L = ctypes.CDLL(str(_lib.lib_path()))
    L.atb_noalloc_last_error.restype = ctypes.c_char_p
    return L


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _regular(L, dy, x, w, rstd, dt):
    M, N = x.shape
    parts = L.atb_norm_bwd_parts(ctypes.c_int(M))
    pdw = torch.empty(parts, N, dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.atb_norm_bwd(_p(dy), _p(x), _p(w), _p(None), _p(rstd), _p(None), _p(dx), _p(pdw), _p(None),
                          ctypes.c_int(parts), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(0), ctypes.c_int(dt),
                          st) == 0
    assert L.atb_colsum(_p(pdw), _p(dw), ctypes.c_int(parts), ctypes.c_int(N), ctypes.c_int(dt), ctypes.c_int(0),
                        st) == 0
    return dx, dw


def _noalloc(L, dy, x, w, rstd, dt):
    M, N = x.shape
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.atb_rmsnorm_bwd_noalloc(_p(dy), _p(x), _p(w), _p(rstd), _p(dx), _p(dw), ctypes.c_int(M), ctypes.c_int(N),
                                   ctypes.c_int(dt), st)
    assert rc == 0, L.atb_noalloc_last_error()
    return dx, dw


# size pairs: the second call of each pair is smaller, so stale scratch lies beyond what it writes;
# (5, 8192) sits on the N limit with fewer rows than partial slots, (3, 8) is the smallest legal N
@pytest.mark.parametrize("sizes", [[(777, 4096), (300, 1024)], [(5, 8192), (3, 8)]])
@pytest.mark.parametrize("dtype,dt", [(torch.bfloat16, 0), (torch.float16, 1), (torch.float32, 2)])
def test_noalloc_matches_regular_twice(dtype, dt, sizes):
    L = _raw_lib()
    torch.manual_seed(11)
    for call, (M, N) in enumerate(sizes):
        x = torch.randn(M, N, device="cuda", dtype=dtype)
        dy = torch.randn(M, N, device="cuda", dtype=dtype)
        w = (1 + 0.1 * torch.randn(N, device="cuda")).to(dtype)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        dx_ref, dw_ref = _regular(L, dy, x, w, rstd, dt)
        dx, dw = _noalloc(L, dy, x, w, rstd, dt)
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref), f"call {call}: dx differs"
        tol = 1e-4 if dtype == torch.float32 else 3e-2
        assert torch.allclose(dw.float(), dw_ref.float(), rtol=tol, atol=tol * max(1.0, M ** 0.5)), \
            f"call {call}: dw differs by {(dw.float() - dw_ref.float()).abs().max().item()}"
        # and against plain PyTorch fp32 math
        xh = x.float() * rstd[:, None]
        dw_t = (dy.float() * xh).sum(0)
        assert torch.allclose(dw.float(), dw_t, rtol=tol, atol=tol * max(1.0, M ** 0.5))


def test_noalloc_rejects_oversize():
    L = _raw_lib()
    n_max = L.atb_noalloc_max_n()
    N = n_max + 8
    x = torch.zeros(4, N, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(N, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    rc = L.atb_rmsnorm_bwd_noalloc(_p(x), _p(x), _p(w), _p(rstd), _p(dx), _p(dw), ctypes.c_int(4), ctypes.c_int(N),
                                   ctypes.c_int(0), ctypes.c_void_p(0))
    assert rc != 0
    assert b"exceeds" in L.atb_noalloc_last_error()
