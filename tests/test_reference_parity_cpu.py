"""Numerical parity with the unmodified reference (installed under baseline/_ref) where its code runs on CPU:
the AGD and WSAM optimizers, step by step on the same problem. The reference runs in a clean interpreter whose only
``atorch`` is the reference; this process runs this package; the parameter trajectories are compared."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

_PROBLEM = r"""
import torch, torch.nn as nn


def make():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(6, 8), nn.Tanh(), nn.Linear(8, 3))
    g = torch.Generator().manual_seed(1)
    xs = [torch.randn(5, 6, generator=g) for _ in range(8)]
    ys = [torch.randn(5, 3, generator=g) for _ in range(8)]
    return m, xs, ys


def run(kind, AGD, WeightedSAM, cfg):
    m, xs, ys = make()
    traj = []
    if kind == "agd":
        opt = AGD(m.parameters(), **cfg)
        for x, y in zip(xs, ys):
            opt.zero_grad()
            ((m(x) - y) ** 2).mean().backward()
            opt.step()
            traj.append(torch.cat([p.detach().reshape(-1) for p in m.parameters()]).tolist())
    else:
        base = torch.optim.SGD(m.parameters(), lr=0.1, momentum=0.9)
        opt = WeightedSAM(m, base, **cfg)
        for x, y in zip(xs, ys):
            def closure():
                opt.zero_grad()
                loss = ((m(x) - y) ** 2).mean()
                loss.backward()
                return loss
            opt.step(closure)
            traj.append(torch.cat([p.detach().reshape(-1) for p in m.parameters()]).tolist())
    return traj
"""

_REF_MAIN = _PROBLEM + r"""
import json, sys
import atorch
assert "baseline/_ref" in atorch.__file__.replace("\\", "/"), atorch.__file__
from atorch.optimizers.agd import AGD
from atorch.optimizers.wsam import WeightedSAM
kind, cfg = sys.argv[1], json.loads(sys.argv[2])
print("TRAJ" + json.dumps(run(kind, AGD, WeightedSAM, cfg)))
"""


def _reference(kind, cfg, tmp_path):
    if not os.path.isdir(os.path.join(REF, "atorch")):
        pytest.skip("the reference is not installed under baseline/_ref")
    script = tmp_path / "ref_main.py"
    script.write_text(_REF_MAIN)
    res = subprocess.run([sys.executable, str(script), kind, json.dumps(cfg)], cwd=str(tmp_path),
                         env=dict(os.environ, PYTHONPATH=REF), capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("TRAJ")][-1]
    return torch.tensor(json.loads(line[4:]))


def _ours(kind, cfg):
    from atorch_b200.optimizers import AGD, WeightedSAM

    ns = {}
    exec(_PROBLEM, ns)
    return torch.tensor(ns["run"](kind, AGD, WeightedSAM, cfg))


@pytest.mark.parametrize("cfg", [dict(lr=1e-2), dict(lr=1e-2, weight_decay=0.1, amsgrad=True),
                                 dict(lr=1e-2, weight_decay=0.1, weight_decouple=False, clip=0.5),
                                 dict(lr=1e-2, win=True, weight_decay=0.05)])
def test_agd_follows_the_reference_trajectory(cfg, tmp_path):
    ref, ours = _reference("agd", cfg, tmp_path), _ours("agd", cfg)
    assert ref.shape == ours.shape and torch.allclose(ours, ref, rtol=1e-4, atol=1e-5), (ours - ref).abs().max()


@pytest.mark.parametrize("cfg", [dict(rho=0.05, gamma=0.9), dict(rho=0.1, gamma=0.5, adaptive=True),
                                 dict(rho=0.05, gamma=0.9, decouple=False)])
def test_wsam_follows_the_reference_trajectory(cfg, tmp_path):
    ref, ours = _reference("wsam", cfg, tmp_path), _ours("wsam", cfg)
    assert ref.shape == ours.shape and torch.allclose(ours, ref, rtol=1e-4, atol=1e-5), (ours - ref).abs().max()


_REF_MISC = r"""
import json, sys, torch
import atorch
assert "baseline/_ref" in atorch.__file__.replace("\\", "/"), atorch.__file__
what = sys.argv[1]
out = {}
if what == "masks":
    from atorch.npu.layers import (create_additive_mask_by_breakpoint_mask,
                                   create_additive_pack_mask_by_startpoint_endpoint_mask)
    B, S = 3, 24
    glm = torch.tensor([5, 0, 24])
    pack = torch.tensor([[[0, 10, 18], [6, 14, 24]], [[2, 2, 2], [9, 9, 9]], [[0, 4, 20], [4, 12, 22]]])
    out["glm"] = create_additive_mask_by_breakpoint_mask(B, S, glm)[:, 0].int().tolist()
    out["pack"] = create_additive_pack_mask_by_startpoint_endpoint_mask(B, S, pack)[:, 0].int().tolist()
elif what == "partition":
    from atorch.pipeline_parallel.pipe_partition import get_rank_stage_info
    cases = []
    for total, pp, vpp, style, manual in [(32, 4, 1, "loop", None), (30, 4, 2, "loop", None), (13, 2, 2, "v", None),
                                          (10, 2, 2, "loop", [1, 2, 3, 4]), (12, 4, 1, "loop", {0: 1, 3: 2}),
                                          (9, 3, 2, "v", None)]:
        cases.append([[list(t) for t in get_rank_stage_info(total, r, pp, vpp, style, manual)] for r in range(pp)])
    out["cases"] = cases
elif what == "ewma":
    from atorch.local_sgd.utils.anomaly_detection import OnlineDynamicEWMA
    g = torch.Generator().manual_seed(3)
    xs = (1.0 + 0.1 * torch.randn(60, generator=g)).tolist()
    xs[40], xs[55] = 5.0, 0.2
    d = OnlineDynamicEWMA(alpha=0.1, warmup_steps=10, base_threshold=3)
    rec = []
    for x in xs:
        x = torch.tensor(x)
        flag = bool(d.is_outlier(x))
        if not flag:
            d.update(x)
        rec.append([flag, float(d.get_mean()), float(d.get_std())])
    out["rec"], out["xs"] = rec, xs
elif what == "gating":
    from atorch.modules.moe.topk_gating import topk_gating
    from atorch.modules.moe.switch_gating import switch_gating
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(16, 2, 4, generator=g)
    res = []
    for k, cap, v2 in [(2, -1, False), (2, 3, False), (3, 4, False), (2, 3, True), (3, -1, True)]:
        l, w, d = topk_gating(logits, k=k, capacity=cap, need_l_aux=True, dispatchV2=v2)
        res.append([float(l), w.tolist(), (d[0].tolist() if v2 else d.int().tolist())])
    for cap, v2 in [(-1, False), (2, False), (2, True)]:
        l, w, d = switch_gating(logits, capacity=cap, need_l_aux=True, dispatchV2=v2)
        res.append([float(l), w.tolist(), (d[0].tolist() if v2 else d.int().tolist())])
    out["res"], out["logits"] = res, logits.tolist()
print("OUT" + json.dumps(out))
"""


def _reference_misc(what, tmp_path):
    if not os.path.isdir(os.path.join(REF, "atorch")):
        pytest.skip("the reference is not installed under baseline/_ref")
    script = tmp_path / "ref_misc.py"
    script.write_text(_REF_MISC)
    res = subprocess.run([sys.executable, str(script), what], cwd=str(tmp_path), env=dict(os.environ, PYTHONPATH=REF),
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("OUT")][-1][3:])


def test_glm_masks_equal_the_reference_constructions(tmp_path):
    """Visibility of the GLM break-point mask and of the packed start/end-point mask: the dense mask of this package,
    and the per-row key intervals its flash kernels take, against the reference's own constructions."""
    from atorch_b200.ops import flash
    from atorch_b200.ops.attention import build_dense_mask

    from atorch_b200.npu.layers import (create_additive_mask_by_breakpoint_mask,
                                        create_additive_pack_mask_by_startpoint_endpoint_mask)

    ref = _reference_misc("masks", tmp_path)
    B, S = 3, 24
    glm = torch.tensor([5, 0, 24], dtype=torch.int32)
    pack = torch.tensor([[[0, 10, 18], [6, 14, 24]], [[2, 2, 2], [9, 9, 9]], [[0, 4, 20], [4, 12, 22]]], dtype=torch.int32)
    j = torch.arange(S)
    for key, kw in (("glm", dict(glm_mask=glm)), ("pack", dict(pack_glm_mask=pack))):
        want = torch.tensor(ref[key]).bool()
        dense = build_dense_mask(B, S, S, torch.device("cpu"), True, kw.get("glm_mask"), kw.get("pack_glm_mask"), None, None)
        assert torch.equal(dense.expand(B, -1, S, S)[:, 0], want), key
        lo, hi = flash.row_intervals(B, S, S, torch.device("cpu"), True, kw.get("glm_mask"), kw.get("pack_glm_mask"))
        vis = (j[None, None] >= lo[:, :, None]) & (j[None, None] < hi[:, :, None])
        assert torch.equal(vis, want), key
    assert torch.equal(create_additive_mask_by_breakpoint_mask(B, S, glm.long())[:, 0].bool(), torch.tensor(ref["glm"]).bool())
    assert torch.equal(create_additive_pack_mask_by_startpoint_endpoint_mask(B, S, pack.long())[:, 0].bool(),
                       torch.tensor(ref["pack"]).bool())
    one = create_additive_mask_by_breakpoint_mask(B, S, torch.tensor(5))
    assert one.shape == (1, 1, S, S) and torch.equal(one[0, 0].bool(), torch.tensor(ref["glm"][0]).bool())


def test_pipeline_partition_equals_the_reference(tmp_path):
    from atorch_b200.pipeline_parallel.pipe_partition import get_rank_stage_info

    ref = _reference_misc("partition", tmp_path)["cases"]
    mine = []
    for total, pp, vpp, style, manual in [(32, 4, 1, "loop", None), (30, 4, 2, "loop", None), (13, 2, 2, "v", None),
                                          (10, 2, 2, "loop", [1, 2, 3, 4]), (12, 4, 1, "loop", {0: 1, 3: 2}),
                                          (9, 3, 2, "v", None)]:
        mine.append([[list(t) for t in get_rank_stage_info(total, r, pp, vpp, style, manual)] for r in range(pp)])
    assert mine == ref


def test_online_ewma_outlier_detector_equals_the_reference(tmp_path):
    from atorch_b200.local_sgd.anomaly import OnlineDynamicEWMA

    ref = _reference_misc("ewma", tmp_path)
    d = OnlineDynamicEWMA(alpha=0.1, warmup_steps=10, base_threshold=3)
    for x, (flag, mean, std) in zip(ref["xs"], ref["rec"]):
        x = torch.tensor(x)
        mine = bool(d.is_outlier(x))
        if not mine:
            d.update(x)
        assert mine == flag and abs(float(d.get_mean()) - mean) < 1e-6 and abs(float(d.get_std()) - std) < 1e-6, x
    assert any(r[0] for r in ref["rec"])          # the spike was flagged


def test_prototype_gating_equals_the_reference(tmp_path):
    """M6-T prototype gating (top-k with capacity dropping and the compact dispatch form, switch gating) against the
    reference's functions on the same logits."""
    from atorch_b200.modules.moe.prototype_gating import switch_gating, topk_gating

    ref = _reference_misc("gating", tmp_path)
    logits = torch.tensor(ref["logits"])
    got = []
    for k, cap, v2 in [(2, -1, False), (2, 3, False), (3, 4, False), (2, 3, True), (3, -1, True)]:
        got.append(topk_gating(logits, k=k, capacity=cap, need_l_aux=True, dispatchV2=v2))
    for cap, v2 in [(-1, False), (2, False), (2, True)]:
        got.append(switch_gating(logits, capacity=cap, need_l_aux=True, dispatchV2=v2))
    assert len(got) == len(ref["res"])
    for (l, w, d), (rl, rw, rd) in zip(got, ref["res"]):
        assert abs(float(l) - rl) < 1e-6
        assert torch.allclose(w, torch.tensor(rw), atol=1e-6)
        mine = d[0] if isinstance(d, tuple) else d.int()
        assert torch.equal(mine, torch.tensor(rd).to(mine.dtype))


_REDUCERS = r"""
import json, os, sys, torch
import torch.distributed as dist
import torch.multiprocessing as mp

impl = sys.argv[1]
if impl == "reference":
    import atorch
    assert "baseline/_ref" in atorch.__file__.replace("\\", "/"), atorch.__file__
    from atorch.local_sgd.utils.reduce_methods import GTAReducer, LinearReducer
    from atorch.local_sgd.utils.reduce_methods.sparsify import sparsify
else:
    from atorch_b200.local_sgd.reducers import GTAReducer, LinearReducer, sparsify

CASES = [("linear", dict(normalize=True)), ("linear", dict(normalize=False)),
         ("linear", dict(normalize=True, weight_softmax_temperature=0.5)),
         ("gta", dict(consensus_method="sum")), ("gta", dict(consensus_method="count", int8_mask=True)),
         ("gta", dict(consensus_method=None, normalize=True)), ("gta", dict(consensus_method="sum", normalize=False)),
         ("gta", dict(consensus_method="count", weight_softmax_temperature=2.0))]


def worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    out = []
    for kind, kw in CASES:
        g = torch.Generator().manual_seed(100 + rank)
        a, b = torch.randn(7, 5, generator=g), torch.randn(11, generator=g)
        red = (LinearReducer if kind == "linear" else GTAReducer)(dist.group.WORLD, **kw)
        red.reduce_tensor([a, b], weight=0.5 + rank, step_weight=2.0 - 0.5 * rank, step_weight_ratio=0.25)
        out.append([a.tolist(), b.tolist()])
    if rank == 0:
        g = torch.Generator().manual_seed(9)
        t = torch.randn(40, generator=g)
        q.put({"cases": out, "magnitude": sparsify(t.clone(), 0.3, "magnitude").tolist(), "t": t.tolist()})
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=worker, args=(r, 3, int(sys.argv[2]), q)) for r in range(3)]
    [p.start() for p in ps]
    res = q.get(timeout=240)
    [p.join(60) for p in ps]
    print("OUT" + json.dumps(res))
"""


def _run_reducers(impl, tmp_path, port):
    script = tmp_path / "reducers_case.py"
    script.write_text(_REDUCERS)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=REF if impl == "reference" else root)
    res = subprocess.run([sys.executable, str(script), impl, str(port)], cwd=str(tmp_path), env=env, capture_output=True,
                         text=True, timeout=420)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("OUT")][-1][3:])


def test_local_sgd_reducers_equal_the_reference_on_three_gloo_ranks(tmp_path):
    """Linear and generalised-task-arithmetic reducers (sum / count consensus, int8 mask, softmax weights, step-weight
    blending) on three gloo ranks, and magnitude sparsification, against the reference's classes with the same inputs."""
    if not os.path.isdir(os.path.join(REF, "atorch")):
        pytest.skip("the reference is not installed under baseline/_ref")
    import socket

    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    ref = _run_reducers("reference", tmp_path, ports[0])
    mine = _run_reducers("ours", tmp_path, ports[1])
    assert mine["t"] == ref["t"]
    assert torch.allclose(torch.tensor(mine["magnitude"]), torch.tensor(ref["magnitude"]), atol=0)
    assert len(mine["cases"]) == len(ref["cases"]) == 8
    for i, (m, r) in enumerate(zip(mine["cases"], ref["cases"])):
        for x, y in zip(m, r):
            assert torch.allclose(torch.tensor(x), torch.tensor(y), rtol=1e-5, atol=1e-6), i


_MUP = r"""
import json, sys, torch
from torch import nn
impl, tmp = sys.argv[1], sys.argv[2]
if impl == "reference":
    import atorch
    assert "baseline/_ref" in atorch.__file__.replace("\\", "/"), atorch.__file__
    from atorch import mup
    from atorch.mup.module import MupLinear, MupModule, OutputLayer, QKVLayer, QLayer
    from atorch.mup.optim import MuAdamParamGroupsAdjust, MuSGDParamGroupsAdjust
    from atorch.mup.shape import get_infshapes, make_base_shapes, set_base_shapes
    from atorch.mup import init as minit
else:
    from atorch_b200.mup import (MupLinear, MupModule, OutputLayer, QKVLayer, QLayer, MuAdamParamGroupsAdjust,
                                 MuSGDParamGroupsAdjust, get_infshapes, make_base_shapes, set_base_shapes)
    from atorch_b200.mup import init as minit

SAMPLERS = [("normal", dict(std=0.5)), ("uniform", dict(a=-0.3, b=0.3)), ("xavier_uniform", dict(gain=1.5)),
            ("xavier_normal", {}), ("kaiming_uniform", dict(a=0.1)), ("kaiming_normal", dict(mode="fan_out"))]


class Net(MupModule):
    def __init__(self, width, heads_dim=8):
        super().__init__()
        self.emb = nn.Embedding(11, width)
        self.hidden = nn.ModuleList([MupLinear(width, 2 * width, sampler=s, bias_zero_init=(i % 2 == 0), **kw)
                                     for i, (s, kw) in enumerate(SAMPLERS)])
        self.qkv = QKVLayer(width, 3 * width, sampler="normal", std=0.2)
        self.q = QLayer(width, width)
        self.inp = MupLinear(5, width, sampler="kaiming_normal", bias_zero_init=False)
        self.out = OutputLayer(width, 7, output_mult=2.0, sampler="normal", std=0.1, bias_zero_init=False)
        self.out0 = OutputLayer(width, 3, weight_zero_init=True, bias=False)


def dump(model):
    return {n: p.detach().double().flatten().tolist() for n, p in model.named_parameters()}


out = {}
base, delta = Net(6), Net(12)      # multiples of 3: the reference's QLayer wants three row blocks
table = make_base_shapes(base, delta, savefile=tmp + "/" + impl + ".bsh")
out["file"] = open(tmp + "/" + impl + ".bsh").read().split("\n", 2)[2] if impl == "reference" else None
out["file_lines"] = sorted(l for l in open(tmp + "/" + impl + ".bsh").read().splitlines() if not l.startswith("#"))
for width, how in ((24, "models"), (6, "models"), (18, "file")):
    torch.manual_seed(width)
    m = Net(width)
    if how == "models":
        set_base_shapes(m, base, delta=delta)
    else:
        set_base_shapes(m, tmp + "/" + impl + ".bsh")
    rec = {"infshapes": {n: s.serialize() for n, s in get_infshapes(m).items()},
           "ninf": {n: s.ninf() for n, s in get_infshapes(m).items()},
           "mult": {n: float(s.width_mult()) for n, s in get_infshapes(m).items()}}
    for mode in ("mup", "sp"):
        torch.manual_seed(100 + width)
        m.mup_initial(mode)
        rec[mode] = dump(m)
    x = torch.linspace(-1, 1, 2 * width).reshape(2, width)
    rec["readout"] = m.out(x).detach().double().flatten().tolist()
    sizes = lambda groups: [[round(g["lr"], 12), round(g["weight_decay"], 12), sorted(p.numel() for p in g["params"])]
                            for g in groups if g["params"]]
    rec["adam"] = sizes(MuAdamParamGroupsAdjust(m.parameters(), lr=0.01, weight_decay=0.1))
    rec["adam_nowd"] = sizes(MuAdamParamGroupsAdjust([{"params": list(m.hidden.parameters()), "lr": 0.5},
                                                      {"params": list(m.out.parameters())}], scaled_wd=False, lr=0.01,
                                                     weight_decay=0.2))
    rec["sgd"] = sizes(MuSGDParamGroupsAdjust(m.parameters(), lr=0.1, weight_decay=0.01))
    torch.manual_seed(7)
    t = torch.empty(2 * width, width); t.infshape = m.hidden[0].weight.infshape
    v = torch.empty(width); v.infshape = m.inp.bias.infshape
    rec["trunc"] = minit.trunc_normal_(t, std=0.3, a=-0.5, b=0.5).double().flatten().tolist()
    rec["ones"] = minit.ones_(v).tolist() if v.infshape.ninf() == 1 else None
    out[str(width)] = rec
print("OUT" + json.dumps(out))
"""


def _run_mup(impl, tmp_path):
    script = tmp_path / "mup_case.py"
    script.write_text(_MUP)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=REF if impl == "reference" else root)
    res = subprocess.run([sys.executable, str(script), impl, str(tmp_path)], cwd=str(tmp_path), env=env,
                         capture_output=True, text=True, timeout=420)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("OUT")][-1][3:])


def test_mup_shapes_initialisers_and_optimizer_groups_equal_the_reference(tmp_path):
    """muP end to end on one network (every sampler, q/k/v layers, two readouts): width marks from a base/delta pair
    and from a base-shape file, the weights drawn by ``mup_initial`` in both modes from the same seed, the readout's
    forward, and the (lr, weight decay, members) of the MuAdam / MuSGD groups."""
    if not os.path.isdir(os.path.join(REF, "atorch")):
        pytest.skip("the reference is not installed under baseline/_ref")
    ref, mine = _run_mup("reference", tmp_path), _run_mup("ours", tmp_path)
    assert mine["file_lines"] == ref["file_lines"]
    for width in ("24", "6", "18"):
        r, m = ref[width], mine[width]
        assert m["infshapes"] == r["infshapes"] and m["ninf"] == r["ninf"] and m["mult"] == r["mult"], width
        for mode in ("mup", "sp"):
            assert m[mode].keys() == r[mode].keys()
            for name in r[mode]:
                assert torch.allclose(torch.tensor(m[mode][name]), torch.tensor(r[mode][name]), rtol=1e-6, atol=1e-7), \
                    (width, mode, name)
        assert torch.allclose(torch.tensor(m["readout"]), torch.tensor(r["readout"]), rtol=1e-6, atol=1e-7)
        for key in ("adam", "adam_nowd", "sgd"):
            assert sorted(m[key]) == sorted(r[key]), (width, key, m[key], r[key])
        assert torch.allclose(torch.tensor(m["trunc"]), torch.tensor(r["trunc"]), rtol=1e-6, atol=1e-7)
        assert m["ones"] == r["ones"]


_PPO = r"""
import json, sys, types, torch
impl = sys.argv[1]
if impl == "reference":
    import atorch
    assert "baseline/_ref" in atorch.__file__.replace("\\", "/"), atorch.__file__
    from atorch.rl.ppo_utils.ppo_util import get_advantages_and_returns, get_kl_penalty, get_rewards, loss
    from atorch.rl.model_utils.model_util import (FixedKLController, RunningMoments, findattr, flatten_dict,
                                                  get_tensor_stats, rgetattr, rhasattr, whiten)
else:
    from atorch_b200.rl.ppo_util import get_advantages_and_returns, get_kl_penalty, get_rewards, loss
    from atorch_b200.rl.model_util import (FixedKLController, RunningMoments, findattr, flatten_dict, get_tensor_stats,
                                           rgetattr, rhasattr, whiten)

g = torch.Generator().manual_seed(21)
B, P, R, V = 3, 4, 6, 13
T = P + R
logits, ref_logits = torch.randn(B, T, V, generator=g), torch.randn(B, T, V, generator=g)
samples = torch.randint(0, V, (B, T), generator=g)
attn = torch.ones(B, T, dtype=torch.long)
attn[0, -2:] = 0
attn[2, P - 1:] = 0            # a sample whose response is empty
prompt = types.SimpleNamespace(input_ids=samples[:, :P])
lp, klp, mean_kl, st = get_kl_penalty(logits, ref_logits, samples, prompt, attn, 0.07)
scores = torch.tensor([1.5, -0.5, 2.0])
rewards = get_rewards([k.clone() for k in klp], scores, lp)
out = {"lp": [x.tolist() for x in lp], "klp": [x.tolist() for x in klp], "mean_kl": float(mean_kl), "st": st,
       "rewards": [x.tolist() for x in rewards]}

cfg = types.SimpleNamespace(clip_ratio=False, cliprange=0.2, cliprange_value=0.15, vf_coef=0.7, ent_coef=0.01, gamma=0.97,
                            lam=0.9)
values, old_values = torch.randn(B, R, generator=g), torch.randn(B, R, generator=g)
rew = torch.randn(B, R, generator=g)
for wh in (True, False):
    adv, ret = get_advantages_and_returns(old_values, rew, R, use_whitening=wh, config=cfg)
    out["gae_%s" % wh] = [adv.tolist(), ret.tolist()]
new_lp, old_lp = -torch.rand(B, R, generator=g), -torch.rand(B, R, generator=g)
mask = torch.ones(B, R)
mask[1, 4:] = 0
lg = torch.randn(B, R, V, generator=g)
for clip in (False, True):
    cfg.clip_ratio = clip
    l, stats = loss(new_lp, values, old_lp, old_values, adv, ret, mask, lg, config=cfg)
    out["loss_%s" % clip] = [float(l), flatten_dict(stats)]
out["stats"] = get_tensor_stats(values, mask, mask.sum())
out["whiten"] = [whiten(values).tolist(), whiten(values, shift_mean=False).tolist()]
rm = RunningMoments()
rec = []
for i in range(3):
    m, s = rm.update(torch.randn(17, generator=g) * (i + 1) + i)
    rec.append([float(m), float(s), float(rm.mean), float(rm.std), float(rm.var), float(rm.count)])
out["moments"] = rec
obj = types.SimpleNamespace(a=types.SimpleNamespace(b=types.SimpleNamespace(c=5)))
out["attr"] = [rhasattr(obj, "a.b.c"), rhasattr(obj, "a.x.c"), rgetattr(obj, "a.b.c"), findattr(obj, ("q", "a.b")).c,
               FixedKLController(0.3).value]
print("OUT" + json.dumps(out))
"""


def _run_ppo(impl, tmp_path):
    script = tmp_path / "ppo_case.py"
    script.write_text(_PPO)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=REF if impl == "reference" else root)
    res = subprocess.run([sys.executable, str(script), impl], cwd=str(tmp_path), env=env, capture_output=True, text=True,
                         timeout=420)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("OUT")][-1][3:])


def _same(a, b, path=""):
    if isinstance(a, dict):
        assert a.keys() == b.keys(), path
        for k in a:
            _same(a[k], b[k], path + "/" + str(k))
    elif isinstance(a, (list, tuple)):
        assert len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            _same(x, y, path + "/" + str(i))
    elif isinstance(a, float):
        assert abs(a - b) <= 1e-5 + 1e-5 * abs(b), (path, a, b)
    else:
        assert a == b, (path, a, b)


def test_ppo_step_functions_and_statistics_equal_the_reference(tmp_path):
    """KL penalty slices, rewards, GAE (with and without whitening), the clipped loss with its nested statistics,
    masked tensor statistics, running moments and the dotted-attribute helpers on the same random inputs."""
    if not os.path.isdir(os.path.join(REF, "atorch")):
        pytest.skip("the reference is not installed under baseline/_ref")
    _same(_run_ppo("ours", tmp_path), _run_ppo("reference", tmp_path))
