"""Ulysses, ring and distributed-softmax attention on CPU/gloo against dense attention."""
import torch

from tests.dist_utils import run_distributed


def _sp(rank, world):
    from atorch_b200.distributed import distributed as D
    from atorch_b200.modules.distributed_transformer.distributed_attention import DistributedSelfAttention
    from atorch_b200.ops import attention_reference
    from atorch_b200.parallel.sequence_parallel import RingAttention, UlyssesAttention

    D.create_sequence_parallel_group(world)
    g = D.get_sequence_parallel_group()
    torch.manual_seed(0)
    B, S, H, Dh = 2, 8, 4, 16
    q, k, v = (torch.randn(B, S, H, Dh) for _ in range(3))
    sl = slice(rank * S // world, (rank + 1) * S // world)
    for causal in (True, False):
        ref_q, ref_k, ref_v = (t.clone().requires_grad_() for t in (q, k, v))
        ref = attention_reference(ref_q, ref_k, ref_v, causal=causal)
        ref[:, sl].sum().backward()
        for cls in (UlyssesAttention, RingAttention):
            m = cls(causal=causal)
            m.set_sp(world, rank, g)
            lq, lk, lv = (t[:, sl].clone().requires_grad_() for t in (q, k, v))
            out = m(lq, lk, lv)
            assert torch.allclose(out, ref[:, sl], atol=1e-5), (cls.__name__, causal)
            out.sum().backward()
            # each rank back-propagated its own chunk's loss: q grads are local, k/v grads need all ranks
            assert torch.allclose(lq.grad, ref_q.grad[:, sl], atol=1e-5), (cls.__name__, causal)
    dsa = DistributedSelfAttention(num_micro_q=2, group=g)
    qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
    out = dsa(qh[:, :, sl].contiguous(), kh[:, :, sl].contiguous(), vh[:, :, sl].contiguous())
    ref = attention_reference(q, k, v, causal=False).transpose(1, 2)
    assert torch.allclose(out, ref[:, :, sl], atol=1e-5)


def test_sequence_parallel_attention_gloo():
    run_distributed(_sp, world=2)


def test_zigzag_plan_reproduces_causal_attention():
    """The block plan of the load-balanced ring layout (which query rows meet which key rows of which rank), checked
    with dense per-block attention and the log-sum-exp merge on one process: every rank's merged output equals its
    rows of causal attention over the whole sequence, and every rank computes the same number of block products."""
    import math

    import torch

    from atorch_b200.ops.ring_flash import _plan, zigzag_shard, zigzag_unshard
    from atorch_b200.parallel.sequence_parallel import _attn_with_lse

    torch.manual_seed(0)
    W, B, S, H, D = 4, 2, 64, 2, 16
    q, k, v = (torch.randn(B, S, H, D) for _ in range(3))
    scale = 1.0 / math.sqrt(D)
    ref, _ = _attn_with_lse(q, k, v, True, scale)
    parts = [[zigzag_shard(t, r, W) for t in (q, k, v)] for r in range(W)]
    S_loc = S // W
    outs, work = [], []
    for r in range(W):
        out = torch.zeros(B, S_loc, H, D)
        lse = torch.full((B, H, S_loc), float("-inf"))
        n = 0
        for owner in [r] + [(r - s) % W for s in range(1, W)]:
            for qs, ks, cz in _plan(owner, r, True, True, S_loc):
                o_i, l_i = _attn_with_lse(parts[r][0][:, qs], parts[owner][1][:, ks], parts[owner][2][:, ks], cz, scale)
                new = torch.logaddexp(lse[:, :, qs], l_i)
                w_old = torch.exp(lse[:, :, qs] - new).transpose(1, 2).unsqueeze(-1)
                w_new = torch.exp(l_i - new).transpose(1, 2).unsqueeze(-1)
                out[:, qs] = out[:, qs] * w_old + o_i * w_new
                lse[:, :, qs] = new
                n += (qs.stop - qs.start) * (ks.stop - ks.start)
        outs.append(out)
        work.append(n)
    assert torch.allclose(zigzag_unshard(outs), ref, atol=1e-5)
    assert len(set(work)) == 1, work
