"""Sharded engine over NCCL on 2 GPUs: tiny Llama, bf16 compute, per-unit recompute; the loss curve
must track a single-GPU run over the union batch."""
import pytest
import torch

from tests.dist_utils import run_distributed

pytestmark = pytest.mark.gpu


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
    for name, extra in (("fused", {"fused_comm": True}), ("nccl", None),
                        ("in_backward", {"fused_comm": True, "optimizer_in_backward": True})):
        f = str(tmp_path / f"l_{name}.pt")
        run_distributed(_train_rank, world=2, args=(f, extra), backend="nccl", timeout=300)
        runs[name] = torch.load(f)
    multi = runs["fused"]
    for name in ("nccl", "in_backward"):
        assert max(abs(x - y) for x, y in zip(multi, runs[name])) < 0.03, (name, multi, runs[name])
    torch.cuda.set_device(0)
    res = _build([])
    single = []
    for a, b in zip(_batches(0), _batches(1)):
        ids = torch.cat([a, b]).cuda()
        res.optim.zero_grad()
        loss = res.model(input_ids=ids, labels=ids, return_logits=False)[0]
        loss.backward()
        res.optim.step()
        single.append(loss.item())
    assert max(abs(x - y) for x, y in zip(multi, single)) < 0.08, (multi, single)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fsdp_frozen_and_odd_sizes_two_gpus():
    from tests.test_fsdp_cpu import _frozen_odd

    run_distributed(_frozen_odd, world=2, args=("cuda",), backend="nccl", timeout=300)
