"""Pipeline parallel on CPU/gloo: partition arithmetic, schedule action lists, 1F1B and interleaved
execution against a single-process run."""
import torch
import torch.nn as nn

from atorch_b200.pipeline_parallel.pipe_partition import get_rank_stage_info, layers_per_stage
from atorch_b200.pipeline_parallel.pipe_schedule import interleaved_actions, one_f_one_b_actions
from tests.dist_utils import run_distributed


def test_partition():
    assert layers_per_stage(16, 4) == [4, 4, 4, 4]
    assert layers_per_stage(14, 4) == [4, 4, 3, 3]
    assert layers_per_stage(14, 4, [3, 4, 4, 3]) == [3, 4, 4, 3]
    assert layers_per_stage(14, 4, {0: 3, 3: 3}) == [3, 4, 4, 3]
    assert get_rank_stage_info(14, 1, 2, 2) == [(1, 4, 4), (3, 3, 11)]
    assert get_rank_stage_info(8, 0, 2, 2, style="v") == [(0, 2, 0), (3, 2, 6)]


def test_action_lists_are_complete_and_ordered():
    for pp, n in ((2, 4), (4, 8), (4, 2)):
        for r in range(pp):
            a = one_f_one_b_actions(r, pp, n)
            assert sorted(x for x in a if x[0] == "F") == [("F", 0, m) for m in range(n)]
            assert [x[2] for x in a if x[0] == "B"] == list(range(n))
            for m in range(n):
                assert a.index(("F", 0, m)) < a.index(("B", 0, m))
            inflight = peak = 0
            for k, _, _ in a:
                inflight += 1 if k == "F" else -1
                peak = max(peak, inflight)
            assert peak <= pp - r
    a = interleaved_actions(0, 2, 4, 2)
    assert len(a) == 16 and {x for x in a if x[0] == "F"} == {("F", c, m) for c in range(2) for m in range(4)}


class _Chunk(nn.Module):
    def __init__(self, layer_num, pre, post, start):
        super().__init__()
        g = torch.Generator().manual_seed(1)
        all_w = [torch.randn(8, 8, generator=g) * 0.3 for _ in range(4)]
        self.layers = nn.ModuleList()
        for i in range(start, start + layer_num):
            lin = nn.Linear(8, 8, bias=False)
            lin.weight.data.copy_(all_w[i])
            self.layers.append(lin)

    def forward(self, x):
        for l in self.layers:
            x = torch.tanh(l(x))
        return x


def _provider(model_config, layer_num, pre_process, post_process, start_layer_idx):
    return _Chunk(layer_num, pre_process, post_process, start_layer_idx)


def _run_pipe(rank, world, vpp, sche, out_file):
    from atorch_b200.distributed import distributed as D
    from atorch_b200.pipeline_parallel.pipe_module import PipeModuleConfig, make_pipe_module
    from atorch_b200.pipeline_parallel.pipe_schedule import make_pipe_schedule_from_pipe_module

    D.create_parallel_group(([("pipe", world)], None))
    cfg = PipeModuleConfig(total_layer_num=4, virtual_pp_size=vpp, sche_name=sche, n_microbatches=4, auto_ddp=False)
    pm = make_pipe_module(model_provider=_provider, loss_func=lambda o, t: ((o - t) ** 2).mean(), config=cfg)
    sched = make_pipe_schedule_from_pipe_module(pm, cfg)
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(8, 8, generator=g), torch.randn(8, 8, generator=g)
    first = pm.stage_ids[0] == 0
    last = (pm.num_stages - 1) in pm.stage_ids
    if first and last:
        loss = sched.step(x, target=y)
    elif first:
        loss = sched.step(x)
    elif last:
        loss = sched.step(target=y)
    else:
        loss = sched.step()
    grads = {}
    for m, sid in zip(pm.stage_modules, pm.stage_ids):
        for i, l in enumerate(m.layers):
            grads[(sid, i)] = l.weight.grad.clone()
    torch.save({"loss": None if loss is None else loss.item(), "grads": grads, "ids": pm.stage_ids},
               f"{out_file}.{rank}")


def _reference():
    m = _Chunk(4, True, True, 0)
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(8, 8, generator=g), torch.randn(8, 8, generator=g)
    losses = []
    for xm, ym in zip(x.chunk(4), y.chunk(4)):
        l = ((m(xm) - ym) ** 2).mean()
        (l / 4).backward()
        losses.append(l.item())
    return sum(losses) / 4, [l.weight.grad for l in m.layers]


def test_schedules_match_single_process(tmp_path):
    ref_loss, ref_grads = _reference()
    for vpp, sche in ((1, "Schedule1F1B"), (1, "ScheduleGPipe"), (2, "ScheduleInterleaved1F1B")):
        f = str(tmp_path / f"p_{vpp}_{sche}")
        run_distributed(_run_pipe, world=2, args=(vpp, sche, f))
        per = 4 // (2 * vpp)
        seen_loss = False
        for r in range(2):
            d = torch.load(f"{f}.{r}")
            if d["loss"] is not None:
                assert abs(d["loss"] - ref_loss) < 1e-5
                seen_loss = True
            for (sid, i), g in d["grads"].items():
                assert torch.allclose(g, ref_grads[sid * per + i], atol=1e-5), (sche, sid, i)
        assert seen_loss


class _Chain(nn.Module):
    """embed -> 4 layers -> norm -> head, the shape `partition_model_from_meta_model` understands."""

    def __init__(self):
        super().__init__()
        self.embed = nn.Linear(8, 8)
        self.layers = nn.ModuleList([nn.Linear(8, 8) for _ in range(4)])
        self.norm = nn.LayerNorm(8)
        self.head = nn.Linear(8, 8)

    def forward(self, x):
        x = self.embed(x)
        for l in self.layers:
            x = l(x)
        return self.head(self.norm(x))


def _run_meta_pipe(rank, world, out_file):
    from atorch_b200.distributed import distributed as D
    from atorch_b200.pipeline_parallel.pipe_module import PipeModuleConfig, make_pipe_module
    from atorch_b200.pipeline_parallel.pipe_schedule import make_pipe_schedule_from_pipe_module

    D.create_parallel_group(([("pipe", world)], None))
    with torch.device("meta"):
        meta = _Chain()
    cfg = PipeModuleConfig(total_layer_num=4, sche_name="Schedule1F1B", n_microbatches=2, auto_ddp=False)
    pm = make_pipe_module(meta_model=meta, loss_func=lambda o, t: ((o - t) ** 2).mean(), config=cfg)
    st = pm.stage_modules[0]
    assert not any(p.is_meta for p in st.parameters())
    if rank == 0:
        assert len(st.pre) == 1 and len(st.layers) == 2 and len(st.post) == 0
    else:
        assert len(st.pre) == 0 and len(st.layers) == 2 and len(st.post) == 2
    # load known weights so that the result can be compared with the unpartitioned model
    torch.manual_seed(5)
    full = _Chain()
    mine = {0: [full.embed, full.layers[0], full.layers[1]], 1: [full.layers[2], full.layers[3], full.norm, full.head]}[rank]
    for dst, src in zip(list(st.pre) + list(st.layers) + list(st.post), mine):
        dst.load_state_dict(src.state_dict())
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(4, 8, generator=g), torch.randn(4, 8, generator=g)
    sched = make_pipe_schedule_from_pipe_module(pm, cfg)
    loss = sched.step(x) if rank == 0 else sched.step(target=y)
    if rank == 1:
        ref = sum(((full(xm) - ym) ** 2).mean() for xm, ym in zip(x.chunk(2), y.chunk(2))) / 2
        assert abs(loss.item() - ref.item()) < 1e-5, (loss.item(), ref.item())
    torch.save(True, f"{out_file}.{rank}")


def test_pipe_module_from_meta_model(tmp_path):
    run_distributed(_run_meta_pipe, world=2, args=(str(tmp_path / "m"),))


def _run_pipe_engine(rank, world, out_file):
    from atorch_b200.distributed import distributed as D
    from atorch_b200.pipeline_parallel.pipe_engine import PipeEngine, PipeSchedulerType, is_batch_on_device
    from atorch_b200.pipeline_parallel.pipe_module import PipeModuleConfig, make_pipe_module

    D.create_parallel_group(([("pipe", world)], None))
    with torch.device("meta"):
        meta = _Chain()
    cfg = PipeModuleConfig(total_layer_num=4, sche_name="Schedule1F1B", n_microbatches=2, auto_ddp=False)
    pm = make_pipe_module(meta_model=meta, loss_func=lambda o, t: ((o - t) ** 2).mean(), config=cfg)
    st = pm.stage_modules[0]
    torch.manual_seed(5)
    full = _Chain()
    mine = {0: [full.embed, full.layers[0], full.layers[1]], 1: [full.layers[2], full.layers[3], full.norm, full.head]}[rank]
    for dst, src in zip(list(st.pre) + list(st.layers) + list(st.post), mine):
        dst.load_state_dict(src.state_dict())
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(8, 8, generator=g), torch.randn(8, 8, generator=g)
    batches = [(x[i: i + 2], y[i: i + 2]) for i in range(0, 8, 2)]
    assert is_batch_on_device(batches, "cpu") and is_batch_on_device({"a": [x, 3]}, "cpu")
    for sched, avg in (("OneForwardOneBackward", False), ("ForwardBackwardNoPipelinging", True)):
        eng = PipeEngine(pm, {"scheduler": sched, "global_batchsize": 8, "micro_batchsize": 2, "device": "cpu",
                              "return_average_loss": avg})
        assert eng.config.scheduler is PipeSchedulerType(sched) and eng.n_microbatches == 4
        assert eng.config.virtual_pp_size == 1
        for p in st.parameters():
            p.grad = None
        out = eng.train_batch_step(iter(batches))
        ref = [((full(xm) - ym) ** 2).mean() for xm, ym in batches]
        if rank == world - 1:
            if avg:
                assert abs(out.item() - (sum(ref) / 4).item()) < 1e-5
            else:
                assert len(out) == 4 and all(abs(a.item() - b.item()) < 1e-5 for a, b in zip(out, ref))
        else:
            assert out == []
        full.zero_grad()
        (sum(ref) / 4).backward()
        for dst, src in zip(list(st.pre) + list(st.layers) + list(st.post), mine):
            for a, b in zip(dst.parameters(), src.parameters()):
                assert torch.allclose(a.grad, b.grad, atol=1e-5)
    torch.save(True, f"{out_file}.{rank}")


def test_pipe_engine_runs_a_step_from_a_data_iterator(tmp_path):
    f = str(tmp_path / "engine")
    run_distributed(_run_pipe_engine, world=2, args=(f,))
    assert all(torch.load(f"{f}.{r}") for r in range(2))
