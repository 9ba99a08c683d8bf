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


def test_fx_meta_tools_and_mip_tensor_parallel_planner():
    """Trace a transformer block, propagate shapes on meta tensors, solve the layout MIP: large layers pair
    column→row (attention and MLP), tiny layers stay replicated, a memory budget forces sharding, and the
    sharding-spec propagation names the collectives the chosen layout needs."""
    import torch
    import torch.nn as nn

    from atorch_b200.auto.mip_tp_planner import MIPTensorParallelPlanner
    from atorch_b200.utils.shape_prop import MetaShapeProp
    from atorch_b200.utils.sharding_spec import MeshShardingSpec, reshard_plan
    from atorch_b200.utils.spec_prop import SpecProp
    from atorch_b200.utils.tracer import trace_model

    class Block(nn.Module):
        def __init__(self, h, f, heads):
            super().__init__()
            self.h, self.heads = h, heads
            self.ln1, self.ln2 = nn.LayerNorm(h), nn.LayerNorm(h)
            self.q, self.k, self.v, self.o = (nn.Linear(h, h) for _ in range(4))
            self.up, self.down = nn.Linear(h, f), nn.Linear(f, h)

        def forward(self, x):
            b, s, _ = x.shape
            y = self.ln1(x)
            q, k, v = (l(y).view(b, s, self.heads, -1).transpose(1, 2) for l in (self.q, self.k, self.v))
            a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + self.o(a.transpose(1, 2).reshape(b, s, self.h))
            return x + self.down(torch.nn.functional.gelu(self.up(self.ln2(x))))

    big = Block(4096, 16384, 32)
    gm = trace_model(big)
    MetaShapeProp(gm).propagate(torch.empty(2, 2048, 4096, device="meta"))
    up = next(n for n in gm.graph.nodes if n.target == "up")
    assert up.meta["shape"] == (2, 2048, 16384) and up.meta["flops"] == 2.0 * 2 * 2048 * 16384 * 4096
    assert up.meta["module_path"] == "up"
    plan = MIPTensorParallelPlanner(tp_size=4).plan_graph(gm)
    assert plan == {"q": "col", "k": "col", "v": "col", "o": "row", "up": "col", "down": "row"}, plan
    sp = SpecProp(gm, plan)
    sp.propagate()
    kinds = sorted(op for _, _, ops in sp.conversions for op in ops)
    assert kinds == ["all_reduce", "all_reduce"], sp.conversions          # one per row-parallel output
    # tiny layers: communication outweighs the saved compute
    small = Block(64, 128, 4)
    plan_s = MIPTensorParallelPlanner(tp_size=4).plan(small, (torch.empty(1, 16, 64),))
    assert set(plan_s.values()) == {"replicate"}, plan_s
    # ... unless the parameters do not fit unsharded
    total = sum(p.numel() * 4 for n, p in small.named_parameters() if "ln" not in n)
    plan_m = MIPTensorParallelPlanner(tp_size=4, memory_budget_bytes=0.3 * total).plan(small, (torch.empty(1, 16, 64),))
    assert sum(v != "replicate" for v in plan_m.values()) >= 5, plan_m
    # conversions between specs
    S, R, P = MeshShardingSpec.split(3, -1), MeshShardingSpec.replicated(3), MeshShardingSpec((-1, -1, -1), (0,))
    assert reshard_plan(S, R) == ["all_gather"] and reshard_plan(R, S) == [] and reshard_plan(P, R) == ["all_reduce"]
    assert reshard_plan(P, S) == ["reduce_scatter"] and reshard_plan(S, MeshShardingSpec.split(3, 1)) == ["all_to_all"]
    assert S.shard_shape((2, 8, 64), (4,)) == (2, 8, 16)
