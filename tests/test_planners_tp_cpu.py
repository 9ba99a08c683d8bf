"""Dim planner / pipeline partition DP, automatic tensor-parallel plan + apply (gloo), sharded local SGD (gloo)."""
import torch
import torch.nn as nn

from atorch_b200.auto.planner import DimPlanner, SimpleTopology, tera_pipe_partition
from tests.dist_utils import run_distributed


def test_tera_pipe_partition_and_topology():
    assert tera_pipe_partition([1, 1, 1, 1], [1, 1, 1, 1], 2) == [2, 2]
    sizes = tera_pipe_partition([4, 1, 1, 1, 1], [1] * 5, 2)
    assert sizes == [1, 4]
    assert tera_pipe_partition([1, 1, 1], [5, 5, 5], 1, mem_cap=6) is None
    topo = SimpleTopology(2, 8, 900e9, 50e9)
    assert topo.effective_bandwidth([0, 1, 7]) == 900e9 and topo.effective_bandwidth([0, 8]) == 50e9
    assert topo.all_reduce_time(1e9, [0]) == 0.0


def test_dim_planner_prefers_data_parallel_when_it_fits():
    m = nn.Sequential(*[nn.Linear(256, 256) for _ in range(8)])
    plan = DimPlanner(num_nodes=1, num_devices_per_node=8, memory_bound=10e9, flops=1.4e15).generate_sharding_plan(m)
    assert plan["tensor"] * plan["pipe"] * plan["data"] == 8 and plan["tensor"] == 1 and plan["pipe"] == 1
    tight = DimPlanner(num_nodes=1, num_devices_per_node=8, memory_bound=1.5e6, flops=1.4e15) \
        .generate_sharding_plan(m, activation_bytes_per_layer=1e3)
    assert tight["tensor"] * tight["pipe"] > 1


def _tp_llama(rank, world):
    from atorch_b200.auto import auto_accelerate
    from atorch_b200.distributed import distributed as D
    from atorch_b200.models.llama import LlamaConfig, LlamaModel
    from atorch_b200.modules.distributed_modules import ColumnParallelLinear, RowParallelLinear
    from atorch_b200.parallel.tensor_parallel import plan_tensor_parallel

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=16)
    ref = LlamaModel(cfg)
    ids = torch.randint(0, 64, (2, 16))
    ref_loss, _ = ref(ids, labels=ids)
    model = LlamaModel(cfg)
    model.load_state_dict(ref.state_dict())
    ok, res, _ = auto_accelerate(model, load_strategy=[("parallel_mode", ([("tensor", world)], None)),
                                                       ("tensor_parallel", None)])
    assert ok
    m = res.model
    assert isinstance(m.layers[0].qkv_proj, ColumnParallelLinear) and m.layers[0].qkv_proj.stride == 3
    assert isinstance(m.layers[0].down_proj, RowParallelLinear) and m.layers[0].n_q == 4 // world
    loss, _ = m(ids, labels=ids)
    assert abs(loss.item() - ref_loss.item()) < 1e-4, (loss.item(), ref_loss.item())
    loss.backward()
    plan = plan_tensor_parallel(LlamaModel(cfg))
    assert "layers.0.gate_up_proj" in plan["column"] and "layers.1.o_proj" in plan["row"]


def test_auto_tensor_parallel_llama_gloo():
    run_distributed(_tp_llama, world=2)


def _lsgd(rank, world, tmp):
    from atorch_b200.auto import auto_accelerate
    from atorch_b200.local_sgd import LocalSGDConfig, OuterOptimizerConfig
    from atorch_b200.local_sgd.sharded import load_local_sgd_state_dict, save_local_sgd_state_dict

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 4))
    fs = {"atorch_wrap_cls": (nn.Linear,), "use_local_sgd": True,
          "local_sgd_config": LocalSGDConfig(local_sgd_sync_interval=2, local_sgd_warmup_steps=1, clip_pseudo_grad=10.0),
          "outer_optim_config": OuterOptimizerConfig(torch.optim.SGD, {"lr": 0.7, "momentum": 0.9, "nesterov": True})}
    ok, res, _ = auto_accelerate(model, torch.optim.SGD, optim_args={"lr": 0.05},
                                 load_strategy=[("parallel_mode", ([("zero", 2), ("data", 2)], None)), ("fsdp", fs)])
    assert ok and res.model.engine.local_sgd is not None
    eng = res.model.engine
    g = torch.Generator().manual_seed(rank)           # every rank its own data: replicas drift apart
    for step in range(5):
        res.optim.zero_grad()
        res.model(torch.randn(4, 16, generator=g)).pow(2).mean().backward()
        res.optim.step()
        full = torch.cat([v.reshape(-1) for v in res.model.state_dict().values()])
        gathered = [torch.empty_like(full) for _ in range(world)]
        torch.distributed.all_gather(gathered, full)
        same = all(torch.allclose(gathered[0], t, atol=1e-6) for t in gathered)
        # steps 0 (warm-up, synchronous), 1 and 3 (sync points) end with identical replicas
        assert same == (step in (0, 1, 3)), (step, same)
    assert eng.local_sgd.global_step == 5 and eng.local_sgd.outer_steps == 2
    save_local_sgd_state_dict(res.model, save_dir=tmp)
    load_local_sgd_state_dict(res.model, load_dir=tmp)


def test_sharded_local_sgd_gloo(tmp_path):
    run_distributed(_lsgd, world=4, args=(str(tmp_path),))


def test_selective_offload_cpu_passthrough():
    from atorch_b200.auto.opt_lib.checkpoint import apply_checkpoint

    m = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2))
    x = torch.randn(4, 8)
    ref = m(x).sum()
    ref.backward()
    g = m[0].weight.grad.clone()
    m.zero_grad()
    n = apply_checkpoint(m, {"wrap_class": (nn.Linear,), "selective_offload": {"offload_args": [("mm.default", [0])],
                                                                              "num_layers": 2}})
    assert n == 2
    m(x).sum().backward()
    assert torch.allclose(m[0].weight.grad, g)
