"""Fused peer-memory collectives on 2 GPUs against NCCL + PyTorch math."""
import pytest
import torch

from tests.dist_utils import run_distributed

pytestmark = pytest.mark.gpu


def _symm(rank, world):
    import torch.distributed as dist

    from atorch_b200 import ops
    from atorch_b200.parallel.symm import SymmetricBuffer

    dev = torch.device("cuda", rank)
    torch.manual_seed(100 + rank)
    for dtype, n in ((torch.float32, 1 << 20), (torch.bfloat16, 3 * (1 << 20))):
        buf = SymmetricBuffer(n, dtype)
        for it in range(3):
            x = torch.randn(n, device=dev).to(dtype)
            buf.tensor.copy_(x)
            ref = x.float().clone()
            dist.all_reduce(ref)
            buf.all_reduce_(scale=0.5)
            buf.check()
            assert torch.allclose(buf.tensor.float(), ref * 0.5, rtol=2e-2, atol=2e-2), (dtype, it)
    # reduce-scatter + AdamW
    n = 1 << 20
    sl = n // world
    gbuf = SymmetricBuffer(n, torch.bfloat16)
    master = torch.randn(sl, device=dev)
    m, v = torch.zeros(sl, device=dev), torch.zeros(sl, device=dev)
    lp = torch.empty(sl, device=dev, dtype=torch.bfloat16)
    mr, m2, v2 = master.clone(), m.clone(), v.clone()
    for step in range(1, 4):
        g = torch.randn(n, device=dev).to(torch.bfloat16)
        gbuf.tensor.copy_(g)
        gsum = g.float().clone()
        dist.all_reduce(gsum)
        gbuf.reduce_scatter_adamw(master, m, v, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=1.0 / world)
        gbuf.check()
        ops.adamw_reference(mr, m2, v2, gsum[rank * sl:(rank + 1) * sl], None, 1e-2, 0.9, 0.95, 1e-8, 0.1, step,
                            grad_scale=1.0 / world)
        assert torch.allclose(master, mr, rtol=1e-4, atol=1e-4), step
    assert torch.allclose(lp.float(), mr.bfloat16().float(), atol=2e-2)
    out = torch.zeros(sl, device=dev)
    gbuf.reduce_scatter_into(out, scale=1.0 / world)
    gbuf.check()
    assert torch.allclose(out, gsum[rank * sl:(rank + 1) * sl] / world, rtol=1e-3, atol=1e-3)
    # outer Nesterov step
    n = 1 << 18
    sl = n // world
    pbuf = SymmetricBuffer(n, torch.float32)
    torch.manual_seed(5)
    init = torch.randn(n, device=dev)
    synced = init[rank * sl:(rank + 1) * sl].clone()
    mom = torch.zeros(sl, device=dev)
    ref_synced, ref_mom = init.clone(), torch.zeros(n, device=dev)
    for t in range(3):
        torch.manual_seed(1000 * t + rank)
        cur = (ref_synced + 0.01 * torch.randn(n, device=dev))       # this replica's parameters after H inner steps
        pbuf.tensor.copy_(cur)
        mean = cur.clone()
        dist.all_reduce(mean)
        mean /= world
        pbuf.allreduce_nesterov(synced, mom, 0.7, 0.9, True, t == 0)
        pbuf.check()
        pg = ref_synced - mean
        ref_mom = pg.clone() if t == 0 else 0.9 * ref_mom + pg
        ref_synced = ref_synced - 0.7 * (pg + 0.9 * ref_mom)
        assert torch.allclose(pbuf.tensor, ref_synced, rtol=1e-4, atol=1e-5), t
        assert torch.allclose(synced, ref_synced[rank * sl:(rank + 1) * sl], rtol=1e-4, atol=1e-5)
    # all-gather
    sbuf = SymmetricBuffer(4096, torch.bfloat16)
    sbuf.tensor.fill_(float(rank + 1))
    full = torch.empty(4096 * world, device=dev, dtype=torch.bfloat16)
    sbuf.all_gather_into(full)
    sbuf.check()
    for r in range(world):
        assert (full[r * 4096:(r + 1) * 4096] == r + 1).all()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symmetric_fused_collectives():
    run_distributed(_symm, world=min(torch.cuda.device_count(), 4), backend="nccl", timeout=300)
