"""Tensor-parallel layers, mappings, vocabulary-parallel loss and manual sharding on CPU/gloo (world 2)."""
import torch
import torch.distributed as dist
import torch.nn as nn

from tests.dist_utils import run_distributed


def _layers(rank, world):
    from atorch_b200.distributed import distributed as D
    from atorch_b200.modules.distributed_modules import (ColumnParallelLinear, RowParallelLinear,
                                                         VocabParallelEmbedding, vocab_parallel_cross_entropy)

    D.create_parallel_group(([("tensor", world)], None))
    torch.manual_seed(0)
    fc1, fc2 = nn.Linear(16, 32), nn.Linear(32, 16)
    emb = nn.Embedding(20, 16)
    x_ids = torch.randint(0, 20, (3, 6))
    ref_h = emb(x_ids)
    ref = fc2(torch.relu(fc1(ref_h)))
    ref.sum().backward()
    for sp in (False, True):
        col = ColumnParallelLinear(orig_module=fc1, sequence_parallel=sp)
        row = RowParallelLinear(orig_module=fc2, sequence_parallel=sp)
        vemb = VocabParallelEmbedding(orig_module=emb)
        h = vemb(x_ids)
        assert torch.allclose(h, ref_h, atol=1e-6)
        if sp:          # activations are sharded along the sequence dim outside the block
            out = row(torch.relu(col(h.chunk(world, dim=1)[rank].contiguous())))
            assert torch.allclose(out, ref.chunk(world, dim=1)[rank], atol=1e-5)
            out.sum().backward()
            # every rank back-propagated only its sequence shard of the loss: weight grads are partial sums
            for t, full in ((col.weight.grad, fc1.weight.grad.chunk(world, 0)[rank]),
                            (row.weight.grad, fc2.weight.grad.chunk(world, 1)[rank])):
                assert torch.allclose(t, full, atol=1e-5)
            continue
        out = row(torch.relu(col(h)))
        assert torch.allclose(out, ref, atol=1e-5)
        out.sum().backward()
        assert torch.allclose(col.weight.grad, fc1.weight.grad.chunk(world, 0)[rank], atol=1e-5)
        assert torch.allclose(row.weight.grad, fc2.weight.grad.chunk(world, 1)[rank], atol=1e-5)
        assert torch.allclose(vemb.weight.grad, emb.weight.grad.chunk(world, 0)[rank], atol=1e-5)
    # fused q|k|v style: stride 3
    qkv = nn.Linear(8, 12, bias=False)
    c3 = ColumnParallelLinear(orig_module=qkv, stride=3, gather_output=False)
    xx = torch.randn(2, 8)
    full = qkv(xx).view(2, 3, 4)
    mine = c3(xx).view(2, 3, 2)
    assert torch.allclose(mine, full[:, :, rank * 2:(rank + 1) * 2], atol=1e-6)
    # vocabulary-parallel cross entropy vs dense
    logits = torch.randn(7, 20, requires_grad=True)
    labels = torch.randint(0, 20, (7,))
    labels[2] = -100
    dense = nn.functional.cross_entropy(logits, labels, reduction="none", ignore_index=-100)
    dense.sum().backward()
    local = logits.detach()[:, rank * 10:(rank + 1) * 10].clone().requires_grad_()
    lp = vocab_parallel_cross_entropy(local, labels)
    assert torch.allclose(lp, dense, atol=1e-5)
    lp.sum().backward()
    assert torch.allclose(local.grad, logits.grad[:, rank * 10:(rank + 1) * 10], atol=1e-5)


def test_tp_layers_gloo():
    run_distributed(_layers, world=2)


def _mappings(rank, world):
    from atorch_b200.modules.distributed_modules import (collect_and_reshard, gather_from_group, scatter_to_group,
                                                         split_first_dim_gather_last_dim,
                                                         split_last_dim_gather_first_dim)

    full = torch.arange(24, dtype=torch.float32).view(4, 6)
    mine = scatter_to_group(full.clone().requires_grad_(), None, dim=1)
    assert torch.equal(mine, full[:, rank * 3:(rank + 1) * 3])
    assert torch.equal(gather_from_group(mine, None, dim=1), full)
    rows = full.chunk(world, 0)[rank].contiguous()                 # [2, 6] row shard
    swapped = split_last_dim_gather_first_dim(rows, None)          # -> [4, 3] column shard
    assert torch.equal(swapped, full[:, rank * 3:(rank + 1) * 3])
    assert torch.equal(split_first_dim_gather_last_dim(swapped, None), rows)
    assert torch.equal(collect_and_reshard(rows, 0, 1, None), full[:, rank * 3:(rank + 1) * 3])


def test_mappings_gloo():
    run_distributed(_mappings, world=2)


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.wte = nn.Embedding(16, 8)
        self.c_fc = nn.Linear(8, 32)
        self.c_proj = nn.Linear(32, 8)
        self.drop = nn.Dropout(0.0)

    def forward(self, ids):
        return self.drop(self.c_proj(torch.relu(self.c_fc(self.wte(ids)))))


def _manual(rank, world):
    from atorch_b200.distributed import distributed as D
    from atorch_b200.modules.distributed_modules import (ColumnParallelLinear, RowParallelLinear,
                                                         VocabParallelEmbedding)
    from atorch_b200.tensor_parallel.manual_tp import TPInfo, tp_manual_shard

    D.create_parallel_group(([("tensor", world)], None))
    torch.manual_seed(0)
    m = _Block()
    ids = torch.randint(0, 16, (2, 4))
    ref = m(ids)
    info = TPInfo()
    info.shard_col("c_fc")
    info.shard_row("c_proj")
    info.shard_vocab("wte")
    info.replic_drop("drop")
    tp_manual_shard(m, info)
    assert isinstance(m.c_fc, ColumnParallelLinear) and isinstance(m.c_proj, RowParallelLinear)
    assert isinstance(m.wte, VocabParallelEmbedding) and info.is_vocab_parallelled()
    assert torch.allclose(m(ids), ref, atol=1e-5)


def test_manual_tp_gloo():
    run_distributed(_manual, world=2)


def _tp_sp_chunk(rank, world):
    """Sequence-parallel tensor parallelism of a Llama chunk: same loss as the unsharded chunk, and after
    ``sync_sequence_parallel_grads`` the normalisation weights carry the full gradient."""
    from atorch_b200.benchmarks.hybrid_bench import LlamaChunk
    from atorch_b200.distributed import distributed as D
    from atorch_b200.models.llama import LlamaConfig, RMSNorm, causal_lm_loss
    from atorch_b200.parallel.tensor_parallel import (apply_tensor_parallel, mark_sequence_parallel_replicated,
                                                      sync_sequence_parallel_grads)

    D.create_parallel_group(([("tensor", world)], None))
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=16)
    torch.manual_seed(0)
    ref = LlamaChunk(cfg, 2, True, True, 0)
    torch.manual_seed(0)
    m = LlamaChunk(cfg, 2, True, True, 0, sp=True)
    m.load_state_dict(ref.state_dict())
    apply_tensor_parallel(m, {"sequence_parallel": True})
    assert mark_sequence_parallel_replicated(m, (RMSNorm,)) == 5
    ids = torch.randint(0, 64, (1, 16), generator=torch.Generator().manual_seed(1))
    l_ref = causal_lm_loss(ref(ids), ids)
    l_ref.backward()
    loss = causal_lm_loss(m(ids), ids)
    assert abs(loss.item() - l_ref.item()) < 1e-5, (loss.item(), l_ref.item())
    loss.backward()
    partial = m.norm.weight.grad.clone()
    sync_sequence_parallel_grads(m)
    assert torch.allclose(m.norm.weight.grad, ref.norm.weight.grad, atol=1e-5)
    assert not torch.allclose(partial, ref.norm.weight.grad, atol=1e-5)
    assert torch.allclose(m.layers[1].input_layernorm.weight.grad, ref.layers[1].input_layernorm.weight.grad, atol=1e-5)


def test_sequence_parallel_chunk_gloo():
    run_distributed(_tp_sp_chunk, world=2)


def _megatron_blocks(rank, world):
    """GPT-2 (pre-LN, fused Conv1D qkv) and BERT (post-LN) layers of Hugging Face, split over two ranks, must give the
    outputs and input gradients of the unsharded layers; checkpointing with RNG replay must reproduce dropout."""
    import torch.nn as nn
    from transformers import BertConfig, GPT2Config
    from transformers.models.bert.modeling_bert import BertLayer
    from transformers.models.gpt2.modeling_gpt2 import GPT2Block

    from atorch_b200.distributed import distributed as D
    from atorch_b200.modules.distributed_modules import (ParallelTransformerLayer, spec_from_bert_layer,
                                                         spec_from_gpt2_block, tp_checkpoint)
    from atorch_b200.parallel.randomizer import init_randomizer

    D.create_parallel_group(([("tensor", world)], None))
    init_randomizer(99)
    torch.manual_seed(0)
    x = torch.randn(2, 16, 64)
    # ---- GPT-2
    gcfg = GPT2Config(n_embd=64, n_head=4, n_layer=1, n_positions=32, attn_pdrop=0.0, resid_pdrop=0.0,
                      attn_implementation="eager")
    blk = GPT2Block(gcfg, layer_idx=0).eval()
    par = ParallelTransformerLayer.from_unsharded(spec_from_gpt2_block(blk, gcfg)).eval()
    xr, xp = x.clone().requires_grad_(), x.clone().requires_grad_()
    # the block applies whatever mask it is given (the causal one is built by the model around it)
    causal = torch.full((16, 16), float("-inf")).triu(1)[None, None]
    ref = blk(xr, attention_mask=causal)
    ref = ref[0] if isinstance(ref, tuple) else ref
    out = par(xp)
    assert torch.allclose(out, ref, atol=2e-5), (out - ref).abs().max()
    g = torch.randn_like(ref)
    ref.backward(g)
    out.backward(g)
    assert torch.allclose(xp.grad, xr.grad, atol=2e-5)
    assert par.attention.q_proj.weight.shape == (32, 64) and par.mlp.down_proj.weight.shape == (64, 128)
    # ---- BERT (post-LayerNorm, bidirectional)
    bcfg = BertConfig(hidden_size=64, num_attention_heads=4, intermediate_size=128, hidden_dropout_prob=0.0,
                      attention_probs_dropout_prob=0.0, attn_implementation="eager")
    bl = BertLayer(bcfg).eval()
    bp = ParallelTransformerLayer.from_unsharded(spec_from_bert_layer(bl, bcfg)).eval()
    rb = bl(x)
    rb = rb[0] if isinstance(rb, tuple) else rb
    assert torch.allclose(bp(x), rb, atol=2e-5), (bp(x) - rb).abs().max()
    # ---- checkpoint with RNG replay: hidden dropout on, recomputation must see the same masks
    par.train()
    par.p_drop = 0.3
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    init_randomizer(7)
    ya = par(xa)
    ya.sum().backward()
    init_randomizer(7)
    yb = tp_checkpoint(lambda t: par(t), xb)
    yb.sum().backward()
    assert torch.allclose(ya, yb) and torch.allclose(xa.grad, xb.grad, atol=1e-6)
    # the hidden-dropout mask is shared by the tensor group: every rank produced the same output
    ys = [torch.zeros_like(ya) for _ in range(world)]
    torch.distributed.all_gather(ys, ya.detach())
    assert torch.allclose(ys[0], ys[1])
    del nn


def test_megatron_style_blocks_match_hf_layers_gloo():
    run_distributed(_megatron_blocks, world=2)


def _sharded_weight_ref(rank, world):
    import torch.distributed as dist

    from atorch_b200.ops import tp_fused

    rows, K, M = 6, 10, 7
    torch.manual_seed(3)
    w_full = torch.randn(rows * world, K)
    w_shard = w_full[rank * rows:(rank + 1) * rows].clone().requires_grad_()
    torch.manual_seed(20 + rank)
    x = torch.randn(M, K, requires_grad=True)
    y = tp_fused.sharded_weight_linear(x, w_shard, dist.group.WORLD)
    assert torch.allclose(y, x.detach() @ w_full.t(), atol=1e-5)
    gy = torch.randn(M, rows * world)
    y.backward(gy)
    assert torch.allclose(x.grad, gy @ w_full, atol=1e-5)
    dw = gy.t() @ x.detach()
    dist.all_reduce(dw)
    assert torch.allclose(w_shard.grad, dw[rank * rows:(rank + 1) * rows], atol=1e-4)


def test_sharded_weight_linear_reference_form_gloo():
    """Row-sharded weight, every rank its own input: output from the gathered weight, weight gradient summed over
    the ranks and scattered by rows (the contract the fused GPU form is tested against)."""
    from tests.dist_utils import run_distributed

    run_distributed(_sharded_weight_ref, world=2, backend="gloo", timeout=120)


def _tp_activation_checkpoint(rank, world):
    import torch.nn.functional as F

    from atorch_b200.distributed.distributed import create_parallel_group
    from atorch_b200.modules.distributed_modules.activation_checkpointing import (
        TPCheckpointWrapper, checkpoint, gather_split_1d_tensor, get_cuda_rng_tracker, model_parallel_cuda_manual_seed,
        split_tensor_into_1d_equal_chunks, tp_wrap_fn)

    create_parallel_group(([("tensor", world)], None))
    model_parallel_cuda_manual_seed(77)
    tracker = get_cuda_rng_tracker()

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(3)
            self.a, self.b = torch.nn.Linear(8, 16), torch.nn.Linear(16, 8)

        def forward(self, x, scale=1.0, extra=None):
            h = F.dropout(self.a(x), 0.3)                     # default stream
            with tracker.fork():
                h = F.dropout(torch.tanh(h), 0.3)             # model-parallel stream
            return self.b(h) * scale + (0 if extra is None else extra)

    torch.manual_seed(11)
    x = torch.randn(4, 6, 8)                                  # replicated input, first dim divisible by tp
    extra = torch.randn(4, 6, 8)
    chunk = split_tensor_into_1d_equal_chunks(x, new_buffer=True)
    assert chunk.numel() == x.numel() // world
    assert torch.equal(gather_split_1d_tensor(chunk).view_as(x), x)

    def run(wrapped):
        blk = Block()
        mod = tp_wrap_fn(blk) if wrapped else blk
        model_parallel_cuda_manual_seed(77)
        torch.manual_seed(5)
        xi, ei = x.clone().requires_grad_(), extra.clone().requires_grad_()
        y = mod(xi, scale=2.0, extra=ei)
        torch.randn(3)                                        # other random draws between forward and backward
        with tracker.fork():
            torch.randn(3)
        after = torch.get_rng_state().clone(), tracker.get_states()[next(iter(tracker.get_states()))].clone()
        y.square().sum().backward()
        # the recomputation left the streams where the forward pass (and what followed) had put them
        assert torch.equal(torch.get_rng_state(), after[0])
        assert torch.equal(tracker.get_states()[next(iter(tracker.get_states()))], after[1])
        return y.detach(), xi.grad, ei.grad, [p.grad for p in blk.parameters()], mod

    y0, gx0, ge0, gp0, _ = run(False)
    y1, gx1, ge1, gp1, mod = run(True)
    assert isinstance(mod, TPCheckpointWrapper) and mod.a is mod._checkpoint_wrapped_module.a
    assert torch.equal(y0, y1) and torch.allclose(gx0, gx1, atol=1e-6) and torch.allclose(ge0, ge1, atol=1e-6)
    for a, b in zip(gp0, gp1):
        assert torch.allclose(a, b, atol=1e-6)

    # what the checkpoint keeps of the first argument is this rank's slice
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t.numel()) or t, lambda t: t):
        xi = x.clone().requires_grad_()
        y = checkpoint(lambda t, s: torch.tanh(t) * s, True, xi, 3.0)
    assert saved == [x.numel() // world], saved
    y.sum().backward()
    assert torch.allclose(xi.grad, 3.0 * (1 - torch.tanh(x) ** 2), atol=1e-6)
    # without distribution the whole input is kept
    saved.clear()
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t.numel()) or t, lambda t: t):
        checkpoint(lambda t: torch.tanh(t), False, x.clone().requires_grad_())
    assert saved == [x.numel()]
    # the tracker refuses duplicate names and seeds
    import pytest

    with pytest.raises(Exception, match="already exists"):
        tracker.add("model-parallel-rng", 1)
    with pytest.raises(Exception, match="is not added"):
        with tracker.fork("missing"):
            pass


def test_tp_activation_checkpoint_keeps_a_slice_and_replays_rng_gloo():
    run_distributed(_tp_activation_checkpoint, world=2)
