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
