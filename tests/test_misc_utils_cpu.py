"""Small utilities: topology-aware node ranks, memory estimation, sparse all-reduce, module-level numeric checker,
per-stage pipeline checkpoints, dynamic gradient scalers."""
import os
from types import SimpleNamespace

import pytest
import torch
import torch.nn as nn

from tests.dist_utils import run_distributed


def test_rank_reorder_groups_nodes_of_one_switch():
    from atorch_b200.utils.rank_reorder import new_node_rank, reorder_nodes_by_topology

    labels = [{"rack": "r2", "switch": "s1"}, {"rack": "r1", "switch": "s9"}, {"rack": "r2", "switch": "s0"},
              {"rack": "r1", "switch": "s9"}, {}]
    order = reorder_nodes_by_topology(labels)
    assert order == [4, 1, 3, 2, 0]                    # unlabeled first, then rack r1 (stable), then r2 by switch
    assert [new_node_rank(i, labels) for i in range(5)] == [4, 1, 3, 2, 0]
    assert sorted(order) == list(range(5))


def test_estimate_training_memory_scales_with_the_layout():
    from atorch_b200.utils.virtual_optimizer import estimate_training_memory

    m = nn.Linear(1000, 1000, bias=False)               # 1e6 parameters
    one = estimate_training_memory(m)
    assert one == {"params": 2e6, "grads": 4e6, "optimizer_state": 12e6, "total": 18e6}
    eight = estimate_training_memory(m, data=8)
    assert eight["total"] == one["total"] / 8
    zero1 = estimate_training_memory(m, data=8, shard_params=False)
    assert zero1["params"] == 2e6 and zero1["optimizer_state"] == 12e6 / 8
    tp_pp = estimate_training_memory(m, tensor=2, pipe=2)
    assert tp_pp["total"] == one["total"] / 4


def _sparse(rank, world):
    from atorch_b200.utils.sparse import all_reduce_sparse

    idx = torch.tensor([[0, 2], [1, 1]]) if rank == 0 else torch.tensor([[2, 3, 3], [1, 0, 0]])
    val = torch.tensor([1.0, 2.0]) if rank == 0 else torch.tensor([10.0, 5.0, 6.0])
    out = all_reduce_sparse(torch.sparse_coo_tensor(idx, val, (4, 2)))
    dense = torch.zeros(4, 2)
    dense[0, 1], dense[2, 1], dense[3, 0] = 1.0, 12.0, 11.0
    assert torch.equal(out.to_dense(), dense)


def test_all_reduce_sparse_sums_ragged_index_sets():
    run_distributed(_sparse, world=2)


def test_module_numeric_checker_reports_the_module_that_differs(tmp_path):
    from atorch_b200.utils.numeric_checker import module_numeric_checker

    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))
    x = torch.randn(3, 8)
    with module_numeric_checker(m, str(tmp_path), "save"):
        m(x)
    with module_numeric_checker(m, str(tmp_path), "compare") as same:
        m(x)
    assert same.mismatches == []
    with torch.no_grad():
        m[2].weight.add_(0.5)
    with module_numeric_checker(m, str(tmp_path), "compare") as diff:
        m(x)
    names = {d["module"] if "module" in d else d.get("name") for d in diff.mismatches}
    assert names and all(n in ("2", "root") for n in names), diff.mismatches


def _param_with_grad(values):
    p = nn.Parameter(torch.zeros(len(values)))
    p.grad = torch.tensor(values, dtype=torch.float32)
    return p


def test_dynamic_grad_scaler_backs_off_on_overflow_and_grows_after_good_steps():
    from atorch_b200.utils.grad_scaler import BF16GradScaler, DynamicGradScaler

    p = _param_with_grad([8.0, -4.0])
    opt = torch.optim.SGD([p], lr=1.0)
    s = DynamicGradScaler(init_scale=4.0, growth_interval=2)
    assert s.scale(torch.tensor(2.0)).item() == 8.0
    s.step(opt)                                     # gradients are divided by the scale before the update
    assert torch.equal(p.detach(), torch.tensor([-2.0, 1.0])) and not s.has_overflow()
    s.update()
    assert s.get_scale() == 4.0
    p.grad = torch.tensor([1.0, 1.0])
    s.step(opt)
    s.update()
    assert s.get_scale() == 8.0                     # two good steps: the scale grows
    before = p.detach().clone()
    p.grad = torch.tensor([float("inf"), 1.0])
    assert s.step(opt) is None and s.has_overflow() and torch.equal(p.detach(), before)   # step skipped
    s.update()
    assert s.get_scale() == 4.0                     # halved
    sd = s.state_dict()
    t = DynamicGradScaler()
    t.load_state_dict(sd)
    assert t.get_scale() == 4.0
    # bf16: scale pinned to one, only the non-finite check remains
    b = BF16GradScaler()
    assert b.get_scale() == 1.0 and b.scale(torch.tensor(3.0)).item() == 3.0
    p.grad = torch.tensor([float("nan"), 0.0])
    assert b.step(opt) is None and b.has_overflow()
    b.update()
    assert b.get_scale() == 1.0


def test_pipe_grad_scaler_waits_for_every_local_stage():
    from atorch_b200.amp.pipe_amp import PipeGradScaler

    p1, p2 = _param_with_grad([2.0]), _param_with_grad([float("inf")])
    o1, o2 = torch.optim.SGD([p1], lr=1.0), torch.optim.SGD([p2], lr=1.0)
    s = PipeGradScaler(init_scale=2.0, num_local_stages=2)
    try:
        s.step(o1)
        raise AssertionError("stepped before the second local stage was unscaled")
    except RuntimeError:
        pass
    s.unscale_(o2)
    assert s.step(o1) is None and s.step(o2) is None and s.has_overflow()     # one stage overflowed: both skip
    s.update()
    assert s.get_scale() == 1.0
    p1.grad, p2.grad = torch.tensor([2.0]), torch.tensor([4.0])
    s.unscale_(o1)
    s.unscale_(o2)
    s.step(o1)
    s.step(o2)
    assert p1.item() == -2.0 and p2.item() == -4.0


def test_pipe_checkpoint_round_trip(tmp_path):
    from atorch_b200.utils.pipe_file_utils import atorch_load_pipe_checkpoint, atorch_save_pipe_checkpoint

    torch.manual_seed(0)
    stages = [nn.Linear(4, 4), nn.Linear(4, 2)]
    pm = SimpleNamespace(stage_modules=stages, stage_ids=[1, 3], pp_rank=1)
    opt = torch.optim.AdamW([q for m in stages for q in m.parameters()], lr=1e-2)
    sum(m(torch.randn(2, 4)).sum() for m in stages[:1]).backward()
    opt.step()
    atorch_save_pipe_checkpoint(pm, str(tmp_path), opt)
    assert sorted(os.listdir(tmp_path)) == ["pipe_optim_001.pt", "pipe_stage_001.pt", "pipe_stage_003.pt"]
    fresh = [nn.Linear(4, 4), nn.Linear(4, 2)]
    pm2 = SimpleNamespace(stage_modules=fresh, stage_ids=[1, 3], pp_rank=1)
    opt2 = torch.optim.AdamW([q for m in fresh for q in m.parameters()], lr=1e-2)
    atorch_load_pipe_checkpoint(pm2, str(tmp_path), opt2)
    for a, b in zip(stages, fresh):
        assert torch.equal(a.weight, b.weight) and torch.equal(a.bias, b.bias)
    assert opt2.state_dict()["state"][0]["step"] == opt.state_dict()["state"][0]["step"]


def test_ppo_utils_hand_computed_cases():
    from atorch_b200.rl import ppo_utils as P

    logits = torch.log(torch.tensor([[[0.25, 0.75], [0.5, 0.5]]]))
    lp = P.logprobs_of_labels(logits, torch.tensor([[1, 0]]))
    assert torch.allclose(lp, torch.log(torch.tensor([[0.75, 0.5]])), atol=1e-6)
    x = torch.tensor([[1.0, 2.0, 3.0, 100.0]])
    m = torch.tensor([[1.0, 1.0, 1.0, 0.0]])
    w = P.whiten(x, m)
    assert abs((w * m).sum().item()) < 1e-5 and abs(((w ** 2) * m).sum().item() / 3 - 1.0) < 1e-4
    # rewards: KL penalty on every response token, the sequence score on the last one
    r, kl = P.compute_rewards(torch.tensor([2.0]), torch.tensor([[0.0, -1.0, -1.0]]), torch.tensor([[0.0, -2.0, -1.0]]),
                              torch.tensor([[1.0, 1.0, 0.0]]), kl_coef=0.1)
    assert torch.allclose(r, torch.tensor([[0.0, -0.1 + 2.0, 0.0]])) and abs(kl.item() - 1.0) < 1e-6
    # GAE with gamma = lam = 1 and zero values is the reward-to-go
    adv, ret = P.gae(torch.zeros(1, 3), torch.tensor([[1.0, 2.0, 3.0]]), torch.ones(1, 3), gamma=1.0, lam=1.0,
                     use_whitening=False)
    assert torch.equal(adv, torch.tensor([[6.0, 5.0, 3.0]])) and torch.equal(ret, adv)
    # PPO loss: unchanged policy -> ratio 1, no clipping; value loss is half the squared error
    lp0 = torch.tensor([[-1.0, -2.0]])
    loss, stats = P.ppo_loss(lp0, torch.tensor([[1.0, 1.0]]), lp0, torch.tensor([[1.0, 1.0]]), torch.tensor([[1.0, -1.0]]),
                             torch.tensor([[2.0, 1.0]]), torch.ones(1, 2), vf_coef=0.5)
    assert abs(stats["policy_loss"].item()) < 1e-6 and abs(stats["value_loss"].item() - 0.25) < 1e-6
    assert stats["clipfrac"].item() == 0.0 and abs(loss.item() - 0.125) < 1e-6
    # a ratio far above 1 + clip with a positive advantage is clipped
    _, st = P.ppo_loss(torch.tensor([[0.0]]), torch.zeros(1, 1), torch.tensor([[-1.0]]), torch.zeros(1, 1),
                       torch.ones(1, 1), torch.zeros(1, 1), torch.ones(1, 1), cliprange=0.2)
    assert abs(st["policy_loss"].item() + 1.2) < 1e-6 and st["clipfrac"].item() == 1.0


def test_ib_monitor_reads_counters_of_a_fake_sysfs(tmp_path):
    import json
    import time

    from atorch_b200.utils.ib_monitor import IBMonitor, read_counters

    d = tmp_path / "mlx5_0" / "ports" / "1" / "counters"
    d.mkdir(parents=True)
    (d / "port_xmit_data").write_text("1000\n")
    (d / "port_rcv_data").write_text("10\n")
    c = read_counters(str(tmp_path))
    assert c == {"mlx5_0/ports/1/counters/port_xmit_data": 4000, "mlx5_0/ports/1/counters/port_rcv_data": 40}
    out = tmp_path / "ib.json"
    import atorch_b200.utils.ib_monitor as M

    samples = iter([{"p/port_xmit_data": 4000}, {"p/port_xmit_data": 8000}, {"p/port_xmit_data": 8000}])
    real = M.read_counters
    M.read_counters = lambda root: next(samples)          # three successive readings of the counters
    try:
        mon = IBMonitor(interval=0.05, count=2, path=str(out), root=str(tmp_path))
        mon.start()
        time.sleep(0.4)
        mon.stop()
    finally:
        M.read_counters = real
    ev = json.loads(out.read_text())["traceEvents"]
    rates = [e["args"]["bytes_per_s"] for e in ev if e["name"].endswith("port_xmit_data")]
    assert rates == [4000 / 0.05, 0.0] and all(e["ph"] == "C" for e in ev)


def test_safetensors_files_interchange_with_the_safetensors_package(tmp_path):
    """Files written here are read by the `safetensors` package and the other way round; slices are read by seeking."""
    import pytest

    st = pytest.importorskip("safetensors.torch")
    from atorch_b200.utils.safetensors_io import SafeFile, load_file, save_file

    torch.manual_seed(0)
    tensors = {"w": torch.randn(5, 7), "b": torch.randn(7).bfloat16(), "idx": torch.arange(12).view(3, 4),
               "flag": torch.tensor([True, False]), "empty": torch.zeros(0, 3)}
    p = str(tmp_path / "a.safetensors")
    save_file(tensors, p, metadata={"step": 3})
    theirs = st.load_file(p)
    assert set(theirs) == set(tensors) and all(torch.equal(theirs[k], v) for k, v in tensors.items())
    q = str(tmp_path / "b.safetensors")
    st.save_file({k: v for k, v in tensors.items()}, q, metadata={"who": "them"})
    ours = load_file(q)
    assert all(torch.equal(ours[k], v) and ours[k].dtype == v.dtype for k, v in tensors.items())
    f = SafeFile(p)
    assert f.metadata == {"step": "3"} and f.info("w") == (torch.float32, (5, 7))
    assert torch.equal(f.get_slice("w", 8, 20), tensors["w"].reshape(-1)[8:20])
    assert f.get_slice("w", 4, 4).numel() == 0


def test_tensor_inspector_records_activation_and_gradient_statistics():
    from atorch_b200.utils.inspector import TensorInspector, fp8_cosine_similarity, tensor_stats

    s = tensor_stats(torch.tensor([0.0, 2.0, -4.0, float("inf")]))
    assert s["absmax"] == 4.0 and s["zero_frac"] == 0.25 and s["nonfinite_frac"] == 0.25
    assert fp8_cosine_similarity(torch.randn(4, 256)) > 0.99
    m = nn.Sequential(nn.Linear(256, 256), nn.ReLU(), nn.Linear(256, 8))
    ins = TensorInspector(m, module_filter=lambda n, mod: isinstance(mod, nn.Linear), with_fp8=True, interval=2).register()
    for _ in range(3):
        m(torch.randn(4, 256)).sum().backward()
        ins.next_step()
    ins.remove()
    kinds = {(r["module"], r["kind"], r["step"]) for r in ins.records}
    assert kinds == {(n, k, st_) for n in ("0", "2") for k in ("activation", "grad_output") for st_ in (0, 2)}
    assert all("fp8_cos" in r for r in ins.records if r["module"] == "0")
    n = len(ins.records)
    m(torch.randn(4, 256))
    assert len(ins.records) == n                    # hooks removed


def test_dynamic_profiler_follows_its_config_file(tmp_path):
    """A JSON file dropped next to a running job schedules a profiling session some steps ahead; the trace is written
    when the session's steps are over; ranks not named in the file ignore it."""
    import json

    from atorch_b200.utils.dynamic_profiler import DynamicProfiler

    cfg = tmp_path / "profile.json"
    prof = DynamicProfiler(str(cfg), rank=0, start_monitor=False)
    other = DynamicProfiler(str(cfg), rank=3, start_monitor=False)
    for _ in range(2):
        prof.step()
    assert prof.state == prof.IDLE and not prof.monitor.poll_once()
    cfg.write_text(json.dumps({"start_step": 4, "steps": 2, "ranks": [0], "output_dir": str(tmp_path / "out")}))
    assert prof.monitor.poll_once() and prof.state == prof.SCHEDULED
    other.monitor.poll_once()
    assert other.state == other.IDLE
    x = torch.randn(16, 16)
    states = []
    for _ in range(5):
        (x @ x).sum()
        prof.step()
        states.append(prof.state)
    assert states == ["scheduled", "running", "running", "done", "done"]
    trace = prof.session["trace"]
    assert os.path.exists(trace) and "traceEvents" in json.load(open(trace))
    st = json.load(open(tmp_path / ".dynamic_profile_state.0.json"))
    assert st["state"] == "done" and st["step"] == 6
    prof.close()
    other.close()


def _moe_comm(rank, world):
    import torch.distributed as dist

    from atorch_b200.communication.functions import (all_to_all, gather_from_expert_parallel_region_to_moe,
                                                     reduce_scatter_to_expert_parallel_region_from_moe)

    g = dist.group.WORLD
    # uneven all-to-all: rank r sends r + 1 rows to rank 0 and 1 row to rank 1
    x = (torch.arange((rank + 1) + 1, dtype=torch.float32) + 10 * rank).unsqueeze(1).requires_grad_()
    ins = [rank + 1, 1]
    outs = [1, 2] if rank == 0 else [1, 1]
    y = all_to_all(g, x, outs, ins)
    expect = torch.tensor([[0.0], [10.0], [11.0]]) if rank == 0 else torch.tensor([[1.0], [12.0]])
    assert torch.equal(y.detach(), expect)
    (y * (rank + 1)).sum().backward()                    # the backward is the inverse exchange
    assert torch.equal(x.grad, torch.tensor([[1.0], [2.0]]) if rank == 0 else torch.tensor([[1.0], [1.0], [2.0]]))
    # gather / reduce-scatter pair of the expert-parallel region
    t = torch.full((2, 3), float(rank + 1), requires_grad=True)
    gathered = gather_from_expert_parallel_region_to_moe(t, g)
    assert gathered.shape == (4, 3) and torch.equal(gathered[:2].detach(), torch.ones(2, 3))
    gathered.sum().backward()
    assert torch.equal(t.grad, torch.full((2, 3), 2.0))  # every rank's copy of the gathered rows contributes
    u = torch.arange(12, dtype=torch.float32).view(4, 3) * (rank + 1)
    rs = reduce_scatter_to_expert_parallel_region_from_moe(u, g)
    assert torch.equal(rs, (torch.arange(12, dtype=torch.float32).view(4, 3) * 3)[rank * 2:(rank + 1) * 2])


def test_moe_communication_functions_gloo():
    run_distributed(_moe_comm, world=2)


def test_small_utilities_paths_singleton_hooks_metrics_and_graph_helpers(tmp_path):
    import collections

    import torch
    import torch.fx

    from atorch_b200.common.singleton import SingletonMeta
    from atorch_b200.utils.dev_utils import raise_not_impl
    from atorch_b200.utils.graph_transform_utils import combine_map_aggregate, map_aggregate, topo_sort
    from atorch_b200.utils.hooks import ATorchHooks
    from atorch_b200.utils.metric_util import MaskedLM, calc_mlm_acc
    from atorch_b200.utils.path_utils import path_is_empty

    assert path_is_empty(None) and path_is_empty(tmp_path) and path_is_empty(tmp_path / "missing")
    (tmp_path / "f").write_text("x")
    assert not path_is_empty(tmp_path) and path_is_empty(tmp_path / "f")

    class One(metaclass=SingletonMeta):
        def __init__(self, v=1):
            self.v = v

    a = One(5)
    assert One() is a and a.v == 5
    with pytest.raises(AssertionError):
        One(6)

    class Iface:
        @raise_not_impl
        def run(self):
            pass

    with pytest.raises(NotImplementedError, match="Iface does not implement function run"):
        Iface().run()

    seen = []
    fn = lambda *a, **k: seen.append((a, k))      # noqa: E731
    ATorchHooks.register_hook(ATorchHooks.REPORT_METRICS_HOOK, fn)
    ATorchHooks.register_hook(ATorchHooks.REPORT_METRICS_HOOK, fn)
    ATorchHooks.call_hooks(ATorchHooks.REPORT_METRICS_HOOK, 1, x=2)
    ATorchHooks.call_hooks(ATorchHooks.COMPUTE_GPU_UTIL_HOOK, 3)
    ATorchHooks.remove_hook(ATorchHooks.REPORT_METRICS_HOOK, fn)
    ATorchHooks.call_hooks(ATorchHooks.REPORT_METRICS_HOOK, 4)
    assert seen == [((1,), {"x": 2})]

    logits = torch.tensor([[[0.1, 2.0, 0.0], [3.0, 0.0, 0.0], [0.0, 0.0, 1.0], [0.0, 5.0, 0.0]]])
    labels = torch.tensor([[1, -100, 0, 1]])
    assert abs(calc_mlm_acc({"logits": logits}, labels).item() - 2 / 3) < 1e-6
    m = MaskedLM()
    m.record({"logits": logits}, labels)
    m.record({"logits": logits[:, :2]}, labels[:, :2])
    assert abs(m.compute().item() - 3 / 4) < 1e-6

    Pt = collections.namedtuple("Pt", "x y")
    out = map_aggregate({"a": [1, (2, 3)], "p": Pt(4, 5), "s": slice(1, 6, 2)}, lambda v: v * 10)
    assert out == {"a": [10, (20, 30)], "p": Pt(40, 50), "s": slice(10, 60, 20)} and isinstance(out["p"], Pt)
    dst = {"a": [torch.zeros(2), torch.zeros(1)], "b": (torch.zeros(1),)}
    src = {"a": [torch.ones(2), torch.full((1,), 2.0)], "b": (torch.full((1,), 3.0),)}
    res = combine_map_aggregate(dst, src, lambda d, s: d.copy_(s))
    assert res is dst and dst["a"][1].item() == 2.0 and dst["b"][0].item() == 3.0

    class Net(torch.nn.Module):
        def forward(self, x):
            a = x + 1
            b = a * 2
            return a + b

    nodes = list(torch.fx.symbolic_trace(Net()).graph.nodes)
    order = topo_sort(nodes[::-1])
    pos = {n: i for i, n in enumerate(order)}
    assert len(order) == len(nodes) and all(pos[i] < pos[n] for n in nodes for i in n.all_input_nodes)


def test_dataclass_helpers_dump_diff_map_and_keep_unknown_arguments(monkeypatch):
    import enum
    import json
    from dataclasses import dataclass, field

    from atorch_b200.utils.dataclass_utils import (AutoMapperExtraConfigs, DataclassMixin, DynamicDataClass,
                                                   clear_environment, is_json_serializable)

    class Mode(enum.Enum):
        A = "a"
        B = "b"

    def fn():
        pass

    @dataclass
    class Args(DataclassMixin, AutoMapperExtraConfigs):
        steps: int = int(os.environ.get("NO_SUCH_VAR_FOR_TEST", 10))
        mode: Mode = Mode.A
        modes: tuple = (Mode.A, Mode.B)
        hook: object = fn
        nested: dict = field(default_factory=lambda: {"f": fn, "dev": torch.device("cpu")})
        logging_steps: int = 5

    a = Args(steps=20, mode=Mode.B, extra_configs={"log_interval": 7, "other": None})
    d = a.to_dict()
    assert d["mode"] == "b" and d["modes"] == ("a", "b") and d["hook"] == "fn" and d["nested"] == {"f": "fn", "dev": "cpu"}
    assert json.loads(a.to_json_string())["steps"] == 20 and is_json_serializable(d) and not is_json_serializable({1, 2})
    assert a.to_kwargs() == {"steps": 20, "mode": "b", "extra_configs": {"log_interval": 7, "other": None}}
    mapped = a.do_auto_mapping({"logging_steps": "log_interval", "steps": "train_iters", "mode": "other"})
    assert mapped["log_interval"] == 7 and a.logging_steps == 7          # the other system's name wins
    assert mapped["train_iters"] == 20 and mapped["other"] == Mode.B     # filled from the own fields
    assert "train_iters" not in a.extra_configs                          # a copy unless asked to overwrite
    monkeypatch.setenv("ATB_TEST_ENV", "1")
    with clear_environment():
        assert "ATB_TEST_ENV" not in os.environ and not os.environ
    assert os.environ["ATB_TEST_ENV"] == "1"

    @dataclass(init=False)
    class Dyn(DynamicDataClass):
        lr: float = 0.1
        name: str = "x"

    dyn = Dyn(lr=0.5, warmup=3, sched={"k": [1, 2]})
    assert dyn.lr == 0.5 and dyn.name == "x" and dyn.warmup == 3 and dyn.sched == {"k": [1, 2]}
    assert dyn.to_dict() == {"lr": 0.5, "name": "x", "warmup": 3, "sched": {"k": [1, 2]}}
    with pytest.raises(AttributeError):
        dyn.missing
