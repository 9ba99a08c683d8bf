"""Fused peer-memory collectives (csrc/comm.cu) on 2+ GPUs against NCCL + PyTorch math: peer-load and
multimem (NVLS) variants, copy-engine all-gather, stream-ordered flags, and the bounded-wait failure path."""
import pytest
import torch

from tests.dist_utils import run_distributed

pytestmark = pytest.mark.gpu


def _symm(rank, world, nvls):
    import torch.distributed as dist

    from atorch_b200 import ops
    from atorch_b200.parallel import symm
    from atorch_b200.parallel.symm import SymmetricBuffer

    dev = torch.device("cuda", rank)
    torch.manual_seed(100 + rank)

    if nvls and not SymmetricBuffer(64, torch.float32).multicast_ptr:
        return                                     # no multicast address on this system: nothing to test

    def make(n, dtype):
        b = SymmetricBuffer(n, dtype)
        b.use_nvls = bool(nvls)
        return b

    # all-reduce, odd block counts so that the tail handling of the unrolled loops is exercised
    for dtype, n in ((torch.float32, (1 << 20) + 4 * world), (torch.bfloat16, 3 * (1 << 20) + 8 * world)):
        buf = make(n, dtype)
        for it, blocks in enumerate((0, 3, 29)):
            x = torch.randn(n, device=dev).to(dtype)
            buf.wait_peers_done()                  # peers may still read the previous contents
            buf.tensor.copy_(x)
            ref = x.float().clone()
            dist.all_reduce(ref)
            buf.all_reduce_(scale=0.5, max_blocks=blocks)
            buf.check()
            assert torch.allclose(buf.tensor.float(), ref * 0.5, rtol=2e-2, atol=2e-2), (dtype, it)
    # reduce-scatter + AdamW
    n = (1 << 20) + 8 * world
    sl = n // world
    gbuf = make(n, torch.bfloat16)
    master = torch.randn(sl, device=dev)
    m, v = torch.zeros(sl, device=dev), torch.zeros(sl, device=dev)
    lp = torch.empty(sl, device=dev, dtype=torch.bfloat16)
    mr, m2, v2 = master.clone(), m.clone(), v.clone()
    for step in range(1, 4):
        g = torch.randn(n, device=dev).to(torch.bfloat16)
        gbuf.wait_peers_done()
        gbuf.tensor.copy_(g)
        gsum = g.float().clone()
        dist.all_reduce(gsum)
        gbuf.reduce_scatter_adamw(master, m, v, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=1.0 / world,
                                  max_blocks=7 * step)
        gbuf.check()
        ops.adamw_reference(mr, m2, v2, gsum[rank * sl:(rank + 1) * sl], None, 1e-2, 0.9, 0.95, 1e-8, 0.1, step,
                            grad_scale=1.0 / world)
        tol = 2e-2 if nvls else 1e-4               # the switch returns the sum rounded to bf16
        assert torch.allclose(master, mr, rtol=tol, atol=tol), step
        if nvls:                                    # follow the kernel's trajectory for the next step
            mr.copy_(master); m2.copy_(m); v2.copy_(v)
    assert torch.allclose(lp.float(), master.bfloat16().float(), atol=2e-2)
    out = torch.zeros(sl, device=dev)
    gbuf.reduce_scatter_into(out, scale=1.0 / world)
    gbuf.check()
    assert torch.allclose(out, gsum[rank * sl:(rank + 1) * sl] / world, rtol=1e-2 if nvls else 1e-3, atol=2e-2 if nvls else 1e-3)
    out2 = out.clone()
    gbuf.reduce_scatter_into(out2, scale=1.0 / world, accumulate=True, max_blocks=5)
    gbuf.check()
    assert torch.allclose(out2, 2 * out, rtol=1e-5, atol=1e-5)
    # outer Nesterov step
    n = 1 << 18
    sl = n // world
    pbuf = make(n, torch.float32)
    torch.manual_seed(5)
    init = torch.randn(n, device=dev)
    synced = init[rank * sl:(rank + 1) * sl].clone()
    mom = torch.zeros(sl, device=dev)
    ref_synced, ref_mom = init.clone(), torch.zeros(n, device=dev)
    for t in range(3):
        torch.manual_seed(1000 * t + rank)
        cur = (ref_synced + 0.01 * torch.randn(n, device=dev))       # this replica's parameters after H inner steps
        pbuf.wait_peers_done()
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
    if nvls:
        return
    # all-gather: SM kernel and copy engines (the latter ordered by a READY flag)
    sbuf = SymmetricBuffer(4096 + 512, torch.bfloat16)
    sbuf.tensor.fill_(float(rank + 1))
    full = torch.empty(sbuf.numel * world, device=dev, dtype=torch.bfloat16)
    sbuf.all_gather_into(full, max_blocks=3)
    sbuf.check()
    for r in range(world):
        assert (full[r * sbuf.numel:(r + 1) * sbuf.numel] == r + 1).all()
    sbuf.wait_peers_done()
    sbuf.tensor.fill_(float(10 + rank))
    seq = sbuf.signal(symm.CH_READY)
    part = torch.zeros(512 * world, device=dev, dtype=torch.bfloat16)
    sbuf.wait(symm.CH_READY, seq)
    sbuf.copy_engine_all_gather(part, offset=1024, numel=512)
    sbuf.check()
    for r in range(world):
        assert (part[r * 512:(r + 1) * 512] == 10 + r).all()
    dist.barrier()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("nvls", [0, 1])
def test_symmetric_fused_collectives(nvls):
    run_distributed(_symm, world=min(torch.cuda.device_count(), 8), args=(nvls,), backend="nccl", timeout=300)


def _dropped_call(rank, world):
    """A rank that skips one collective call between steps: the others' kernels give up after the
    (shortened) wait limit, report it through the status word and return; after the ranks have agreed
    on the sequence number again on the host, the next call works. Peer loads only (no multimem)."""
    import torch.distributed as dist

    from atorch_b200.parallel import symm
    from atorch_b200.parallel.symm import CommTimeoutError, SymmetricBuffer

    dev = torch.device("cuda", rank)
    n = 1 << 16
    buf = SymmetricBuffer(n, torch.float32)
    buf.use_nvls = False
    out = torch.zeros(n // world, device=dev)
    buf.tensor.fill_(1.0)
    buf.reduce_scatter_into(out)
    buf.check()
    assert (out == world).all()
    dist.barrier()
    symm.set_wait_limit_ns(100_000_000)            # 0.1 s
    timed_out = False
    if rank != world - 1:                          # the last rank never makes this call
        buf.reduce_scatter_into(out)
        try:
            buf.check()
        except CommTimeoutError:
            timed_out = True
        assert timed_out
    torch.cuda.synchronize()
    dist.barrier()                                 # the others learn of it on the host
    buf.resync()
    symm.set_wait_limit_ns(2_000_000_000)
    buf.wait_peers_done()
    buf.tensor.fill_(2.0)
    dist.barrier()
    buf.reduce_scatter_into(out)
    buf.check()
    assert (out == 2 * world).all()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_bounded_wait_reports_and_recovers():
    run_distributed(_dropped_call, world=2, backend="nccl", timeout=120)
