"""Sharded engine on 2, 4 or 8 GPUs (all that the machine has): tiny Llama, bf16 compute, per-unit recompute;
the loss curve must track a single-GPU run over the union batch."""
import pytest
import torch

from tests.dist_utils import run_distributed

pytestmark = pytest.mark.gpu
NGPU = torch.cuda.device_count()
WORLD = 8 if NGPU >= 8 else 4 if NGPU >= 4 else 2


def _cfg():
    from atorch_b200.models.llama import LlamaConfig

    return LlamaConfig(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=3,
                       num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256)


def _batches(rank, steps=6):
    g = torch.Generator().manual_seed(50 + rank)
    return [torch.randint(0, 1024, (2, 256), generator=g) for _ in range(steps)]


def _build(world_strategy, fsdp_extra=None):
    from atorch_b200.auto import auto_accelerate
    from atorch_b200.models.llama import LlamaDecoderLayer, LlamaModel

    torch.manual_seed(0)
    model = LlamaModel(_cfg())
    ok, res, _ = auto_accelerate(
        model, torch.optim.AdamW, loss_func=lambda b, o: o[0], optim_args={"lr": 1e-3, "weight_decay": 0.0},
        load_strategy=world_strategy + [("fsdp", dict({"atorch_wrap_cls": (LlamaDecoderLayer,)}, **(fsdp_extra or {}))),
                                        ("amp_native", {"dtype": torch.bfloat16}),
                                        ("checkpoint", {"wrap_class": (LlamaDecoderLayer,)})])
    assert ok
    return res


def _train_rank(rank, world, out_file, fsdp_extra=None):
    res = _build(["parallel_mode"], fsdp_extra)
    if fsdp_extra and fsdp_extra.get("fused_comm"):
        assert res.model.engine.fused, "the peer-memory collectives were expected to be active"
    dev = torch.device("cuda", rank)
    losses = []
    for ids in _batches(rank):
        ids = ids.to(dev)
        res.optim.zero_grad()
        loss = res.model(input_ids=ids, labels=ids, return_logits=False)[0]
        loss.backward()
        res.optim.step()
        t = loss.detach().clone()
        torch.distributed.all_reduce(t)
        losses.append(t.item() / world)
    if rank == 0:
        torch.save(losses, out_file)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fsdp_two_gpus_tracks_single_gpu(tmp_path):
    runs = {}
    for name, extra in (("fused", {"fused_comm": True}), ("nccl", {"fused_comm": False}),
                        ("in_backward", {"fused_comm": True, "optimizer_in_backward": True})):
        f = str(tmp_path / f"l_{name}.pt")
        run_distributed(_train_rank, world=WORLD, args=(f, extra), backend="nccl", timeout=300)
        runs[name] = torch.load(f)
    multi = runs["fused"]
    for name in ("nccl", "in_backward"):
        assert max(abs(x - y) for x, y in zip(multi, runs[name])) < 0.03, (name, multi, runs[name])
    torch.cuda.set_device(0)
    res = _build([])
    single = []
    for parts in zip(*[_batches(r) for r in range(WORLD)]):
        ids = torch.cat(parts).cuda()
        res.optim.zero_grad()
        loss = res.model(input_ids=ids, labels=ids, return_logits=False)[0]
        loss.backward()
        res.optim.step()
        single.append(loss.item())
    assert max(abs(x - y) for x, y in zip(multi, single)) < 0.08, (multi, single)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fsdp_frozen_and_odd_sizes_two_gpus():
    from tests.test_fsdp_cpu import _frozen_odd

    run_distributed(_frozen_odd, world=WORLD, args=("cuda",), backend="nccl", timeout=300)


def _single_in_backward(out_file, flag):
    torch.cuda.set_device(0)
    from atorch_b200.auto import auto_accelerate
    from atorch_b200.models.llama import LlamaDecoderLayer, LlamaModel

    torch.manual_seed(0)
    ok, res, _ = auto_accelerate(
        LlamaModel(_cfg()), torch.optim.AdamW, loss_func=lambda b, o: o[0], optim_args={"lr": 1e-3},
        load_strategy=[("fsdp", {"atorch_wrap_cls": (LlamaDecoderLayer,), "optimizer_in_backward": flag}),
                       ("amp_native", {"dtype": torch.bfloat16}), ("checkpoint", {"wrap_class": (LlamaDecoderLayer,)})])
    assert ok
    losses = []
    for ids in _batches(0):
        ids = ids.cuda()
        res.optim.zero_grad()
        loss = res.model(input_ids=ids, labels=ids, return_logits=False)[0]
        loss.backward()
        res.optim.step()
        losses.append(loss.item())
    return losses, res


def test_single_gpu_optimizer_in_backward_matches_plain_step():
    """One rank: the per-unit AdamW launched on a side stream during the backward pass gives the same
    trajectory as the single fused step after it; a second backward before step() is refused."""
    a, _ = _single_in_backward(None, False)
    b, res = _single_in_backward(None, True)
    assert res.model.engine._fused_opt is res.optim
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-3, (a, b)
    ids = _batches(0)[0].cuda()
    res.optim.zero_grad()
    res.model(input_ids=ids, labels=ids, return_logits=False)[0].backward()
    with pytest.raises(RuntimeError, match="second backward"):
        res.model(input_ids=ids, labels=ids, return_logits=False)[0].backward()
