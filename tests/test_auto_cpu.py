"""auto_accelerate plumbing on CPU: strategies (list / pickle / file), adjust, search, clip, amp, half."""
import pickle

import torch
import torch.nn as nn

from atorch_b200.auto import Strategy, auto_accelerate, get_strategy, save_strategy
from atorch_b200.auto.analyser import analyse_model
from atorch_b200.auto.clip_grad_norm import clip_grad_norm
from atorch_b200.auto.engine.search import BayesianGenerator, combination_candidates
from atorch_b200.auto.opt_lib import OptimizationLibrary


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc = nn.Linear(32, 32)

    def forward(self, x):
        return torch.relu(self.fc(x)) + x


def model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(16, 32), Block(), Block(), nn.Linear(32, 4))


def data():
    g = torch.Generator().manual_seed(0)
    return [(torch.randn(16, generator=g), int(torch.randint(0, 4, (), generator=g))) for _ in range(64)]


def loss_func(batch, out):
    return nn.functional.cross_entropy(out, batch[1])


def test_strategy_roundtrip(tmp_path):
    ok, s = get_strategy(["parallel_mode", ("amp_native", {"dtype": torch.bfloat16}), ("tensor_parallel", None)])
    assert ok and s.names() == ["parallel_mode", "amp_native", "tensor_parallel"]
    assert s.get("tensor_parallel")[2] is True
    f = tmp_path / "s.pkl"
    save_strategy(s, str(f))
    ok, s2 = get_strategy(str(f))
    assert ok and s2.names() == s.names()
    ok, s3 = get_strategy(pickle.dumps(s))
    assert ok and isinstance(s3, Strategy)
    s.adjust_data_parallel(8)
    assert s.get_parallel_mode() == (True, ([("data", 8)], None))
    lib = OptimizationLibrary()
    assert lib.validate_strategy(s) == (True, [])
    assert lib.validate_strategy(Strategy([("nope", None, False)]))[0] is False
    assert set(lib.opts) >= {"zero1", "zero2", "fsdp", "fsdp2", "parallel_mode", "auto_ddp", "amp_native", "fp8",
                             "tensor_parallel", "module_replace", "checkpoint", "native_dynamo",
                             "pipeline_parallel", "mixed_parallel", "sequence_parallel", "half",
                             "deepspeed_3d_parallel"}


def test_auto_accelerate_variants():
    for strat in (["amp_native"], [("half", "bf16")], [("checkpoint", {"wrap_class": (Block,)})],
                  [("fsdp", {"atorch_wrap_cls": ("Block",)}), ("amp_native", {"dtype": "bf16"})],
                  ["zero1"], ["module_replace"]):
        ok, res, best = auto_accelerate(model(), torch.optim.AdamW, data(), loss_func, optim_args={"lr": 1e-2},
                                        dataloader_args={"batch_size": 16}, load_strategy=strat,
                                        lr_scheduler_cls=torch.optim.lr_scheduler.StepLR,
                                        lr_scheduler_args={"step_size": 1, "gamma": 0.9})
        assert ok, strat
        losses = []
        for b in res.dataloader:
            x = b[0] if res.prepare_input is None else res.prepare_input(b, "cpu")[0]
            res.optim.zero_grad()
            l = res.loss_func(b, res.model(x))
            l.backward()
            res.optim.step()
            res.lr_scheduler.step()
            losses.append(float(l))
        assert all(v == v for v in losses), strat
        assert res.optim.param_groups[0]["lr"] < 1e-2


def test_search_and_analyse():
    a = analyse_model(model())
    assert a["opt_config_submodule_names"] == (Block,) and a["model_params_num"] > 0
    c = combination_candidates(1, a)
    assert len(c) >= 6 and all(s.names()[0] == "parallel_mode" for s in c)
    class TakesBatch(nn.Module):          # model_input_format=None means model(batch)
        def __init__(self):
            super().__init__()
            self.net = model()

        def forward(self, batch):
            return self.net(batch[0])
    ok, res, best = auto_accelerate(TakesBatch(), torch.optim.SGD, data(), loss_func, optim_args={"lr": 1e-2},
                                    dataloader_args={"batch_size": 16}, time_limit=60)
    assert ok and best is not None and res.model is not None
    g = BayesianGenerator(max_iter=6)
    for _ in range(6):
        combo = g.suggest()
        if combo is None:
            break
        g.observe(combo, float(len([x for x in combo if x])))
    assert len(g.tried) >= 4


def test_clip_grad_norm_plain():
    m = model()
    m(torch.randn(8, 16)).sum().backward()
    n = clip_grad_norm(m, 0.1)
    after = torch.sqrt(sum(p.grad.pow(2).sum() for p in m.parameters()))
    assert n > 0.1 and abs(after.item() - 0.1) < 1e-3


def test_engine_executor_state_machine_two_processes():
    """ANALYSE by one process, then per candidate SETUP_PARALLEL_GROUP / DRYRUN by all, WAIT in between,
    FINISH with the fastest candidate; a repeated parallel mode is not set up twice."""
    from atorch_b200.auto.engine.executor import Executor
    from atorch_b200.auto.engine.task import TaskProcessMode, TaskType

    ex = Executor({"node_num": 1, "nproc_per_node": 2})
    t0 = ex.get_task(0)
    assert t0.task_type == TaskType.ANALYSE and t0.process_mode == TaskProcessMode.ONE_PROCESS
    assert ex.get_task(1).task_type == TaskType.WAIT
    ex.report_task_result(t0.task_id, 0, True, {"opt_config_submodule_names": (), "replaceable_pairs": []})
    seen, setups, speed = [], 0, 0.0
    for _ in range(200):
        a, b = ex.get_task(0), ex.get_task(1)
        if a.task_type == TaskType.WAIT and b.task_type == TaskType.WAIT:
            continue
        # an ALL_PROCESS task reaches both processes before either reports
        assert a.task_id == b.task_id and a.process_mode == TaskProcessMode.ALL_PROCESS, (a, b)
        if a.task_type in (TaskType.FINISH, TaskType.FAIL):
            final = a
            break
        if a.task_type == TaskType.SETUP_PARALLEL_GROUP:
            setups += 1
            res = None
        else:
            assert a.task_type == TaskType.DRYRUN
            speed += 1.0
            names = tuple(a.task_info.names())
            seen.append(names)
            res = {"throughput": 100.0 - abs(speed - 3.0)}       # the third candidate is the fastest
        ex.report_task_result(a.task_id, 1, True, res)
        assert ex.get_task(1).task_type == TaskType.WAIT            # process 0 has not reported yet
        ex.report_task_result(a.task_id, 0, True, res)
    assert final.task_type == TaskType.FINISH and tuple(final.task_info.names()) == seen[2]
    assert setups == 1 and len(seen) >= 4 and len(set(seen)) == len(seen)
    assert ex.can_be_terminated
    # every candidate failing ends in FAIL
    ex2 = Executor({"node_num": 1, "nproc_per_node": 1}, time_limit=1000)
    t = ex2.get_task(0)
    ex2.report_task_result(t.task_id, 0, True, {})
    while True:
        t = ex2.get_task(0)
        if t.task_type in (TaskType.FINISH, TaskType.FAIL):
            break
        ex2.report_task_result(t.task_id, 0, t.task_type != TaskType.DRYRUN, {"throughput": 0.0})
    assert t.task_type == TaskType.FAIL


def test_engine_service_round_trip_over_grpc():
    from atorch_b200.auto.engine.service import AccelerationEngine, AutoAccelerationClient, run_worker_loop
    from atorch_b200.auto.engine.task import TaskType

    eng = AccelerationEngine({"node_num": 1, "nproc_per_node": 1}, algo="bo")
    port = eng.start_service(0)
    client = AutoAccelerationClient(f"127.0.0.1:{port}", 0)
    ran = []

    def run_task(task):
        ran.append(task.task_type)
        if task.task_type == TaskType.ANALYSE:
            return True, {"opt_config_submodule_names": ("Linear",), "replaceable_pairs": []}
        if task.task_type == TaskType.DRYRUN:
            return True, {"throughput": 10.0 + ("fsdp" in task.task_info.names()) + 2 * ("amp_native" in task.task_info.names())}
        return True, None
    best = run_worker_loop(client, run_task, poll_interval=0.001)
    client.close()
    eng.tear_down(timeout=5)
    assert ran[0] == TaskType.ANALYSE and ran.count(TaskType.DRYRUN) >= 4
    assert "fsdp" in best.names() and "amp_native" in best.names()


def test_strategy_generation_algorithms_fill_the_executor_stage_by_stage():
    """The combination algorithm adds its whole set in one call; the Bayesian one proposes a candidate per call, learns
    from the throughputs recorded in between and stops by itself; the library hands them out by name."""
    from atorch_b200.auto.engine.executor import Executor, StrategyRecord
    from atorch_b200.auto.engine.sg_algo import (BOAlgorithm, CombinationAlgorithm, StrategyGenerationAlgorithm,
                                                 StrategyGenerationAlgorithmLibrary)

    lib = StrategyGenerationAlgorithmLibrary()
    assert isinstance(lib["combination_sg"], CombinationAlgorithm) and isinstance(lib["bo_sg"], BOAlgorithm)
    assert lib["nope"] is None and StrategyGenerationAlgorithm("x")(None) == (True, None, 0)

    ex = Executor({"node_num": 1, "nproc_per_node": 2})
    ex.analysis = {"opt_config_submodule_names": ("Block",), "replaceable_pairs": ["x"]}
    ex._generate_candidates()
    algo = CombinationAlgorithm()
    done, tasks, n = algo(ex)
    assert done and tasks is None and n == len(ex._candidates) == 9
    assert algo(ex) == (True, None, 0)
    names = {tuple(r.strategy.names()) for r in ex._candidates}
    assert ("parallel_mode",) in names and ("parallel_mode", "module_replace", "amp_native", "fsdp") in names

    ex = Executor({"node_num": 1, "nproc_per_node": 2}, algo="bo")
    ex.analysis = {"opt_config_submodule_names": ("Block",)}
    ex._generate_candidates()
    bo = BOAlgorithm(max_iter=10, patience=3, random_sample=2)
    proposed = []
    for _ in range(40):
        done, _, n = bo(ex)
        if done:
            break
        assert n == 1
        rec = ex._candidates.popleft()
        assert rec.combo not in proposed
        proposed.append(rec.combo)
        rec.status = StrategyRecord.SUCCEED
        rec.dryrun_result = {"throughput": 10.0 + (rec.combo[0] is not None) + 2 * (rec.combo[1] == "fsdp")}
        ex.strategies.append(rec)
    assert bo.is_done and 3 <= len(proposed) <= 10
    best = max(ex.strategies, key=lambda r: r.throughput)
    assert best.combo[1] == "fsdp"                      # the search reached the better zero choice
