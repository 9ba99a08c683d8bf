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
