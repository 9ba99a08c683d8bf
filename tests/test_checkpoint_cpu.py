"""Flat sharded checkpoints: save at world size 2, reload at world size 1, 2 and 4; optimizer state too."""
import torch
import torch.nn as nn

from tests.dist_utils import run_distributed
from tests.test_fsdp_cpu import make_mlp


def _save(rank, world, path, fused):
    from atorch_b200.parallel.fsdp import FSDP, FusedShardedOptimizer, ShardedOptimizer
    from atorch_b200.utils.fsdp_save_util import save_fsdp_flat_param, save_fsdp_optim_param

    f = FSDP(make_mlp(), wrap_cls=(nn.Linear,))
    opt = FusedShardedOptimizer(f.engine, "adamw", lr=1e-3) if fused else \
        ShardedOptimizer(torch.optim.AdamW(f.parameters(), lr=1e-3), f.engine)
    g = torch.Generator().manual_seed(7)
    for _ in range(2):
        opt.zero_grad()
        f(torch.randn(4, 256, generator=g)).sum().backward()
        opt.step()
    save_fsdp_flat_param(f, path)
    save_fsdp_optim_param(f, opt, path)
    if rank == 0:
        torch.save(f.state_dict(), path + "/full_ref.pt")
    else:
        f.state_dict()


def _load(rank, world, path, fused):
    from atorch_b200.parallel.fsdp import FSDP, FusedShardedOptimizer, ShardedOptimizer
    from atorch_b200.utils.fsdp_save_util import ShardOptim, load_fsdp_flat_param

    torch.manual_seed(123)
    m = make_mlp()
    with torch.no_grad():
        for p in m.parameters():
            p.add_(1.0)
    f = FSDP(m, wrap_cls=(nn.Linear,))
    load_fsdp_flat_param(f, path)
    sd = f.state_dict()
    ref = torch.load(path + "/full_ref.pt")
    for k, v in ref.items():
        assert torch.equal(sd[k], v), k
    opt = FusedShardedOptimizer(f.engine, "adamw", lr=1e-3) if fused else \
        ShardedOptimizer(torch.optim.AdamW(f.parameters(), lr=1e-3), f.engine)
    so = ShardOptim(path)
    so.load_into(f, opt)
    # one more identical step must give identical weights on every world size
    g = torch.Generator().manual_seed(99)
    opt.zero_grad()
    f(torch.randn(4, 256, generator=g)).sum().backward()
    opt.step()
    sd2 = f.state_dict()
    if rank == 0:
        torch.save(sd2, path + f"/after_{world}.pt")


def test_flat_checkpoint_reshard(tmp_path):
    for fused in (True, False):
        path = str(tmp_path / f"ckpt_{int(fused)}")
        run_distributed(_save, world=2, args=(path, fused))
        for w in (2, 1, 4):
            run_distributed(_load, world=w, args=(path, fused))
        a2, a1, a4 = (torch.load(path + f"/after_{w}.pt") for w in (2, 1, 4))
        for k in a2:
            assert torch.allclose(a2[k], a1[k], atol=1e-6) and torch.allclose(a2[k], a4[k], atol=1e-6), k


def test_convert_flat_param(tmp_path):
    from atorch_b200.utils.fsdp_save_util import ConvertFlatParam, ShardTensorUtil

    path = str(tmp_path / "c")
    run_distributed(_save, world=2, args=(path, True))
    ref = torch.load(path + "/full_ref.pt")
    sd = ConvertFlatParam(path).convert()
    for k, v in ref.items():
        assert torch.equal(sd[k], v)
    util = ShardTensorUtil(path, name_mapping_func_or_dict={"renamed": "0.weight"})
    assert torch.equal(util.load_tensor_by_name("renamed"), ref["0.weight"])
    assert torch.equal(util.load_param_slice("0.weight", 100, 300), ref["0.weight"].reshape(-1)[100:300])


def _dcp_save(rank, world, path, fused):
    from atorch_b200.parallel.fsdp import FSDP, FusedShardedOptimizer, ShardedOptimizer
    from atorch_b200.utils import dcp_io

    f = FSDP(make_mlp(), wrap_cls=(nn.Linear,))
    opt = FusedShardedOptimizer(f.engine, "adamw", lr=1e-3) if fused else \
        ShardedOptimizer(torch.optim.AdamW(f.parameters(), lr=1e-3), f.engine)
    g = torch.Generator().manual_seed(7)
    for _ in range(2):
        opt.zero_grad()
        f(torch.randn(4, 256, generator=g)).sum().backward()
        opt.step()
    dcp_io.save(f, opt, path, async_save=True)
    dcp_io.wait()
    sd = f.state_dict()
    if rank == 0:
        torch.save(sd, path + "/full_ref.pt")


def _dcp_load(rank, world, path, fused):
    from atorch_b200.parallel.fsdp import FSDP, FusedShardedOptimizer, ShardedOptimizer
    from atorch_b200.utils import dcp_io

    torch.manual_seed(123)
    m = make_mlp()
    with torch.no_grad():
        for p in m.parameters():
            p.add_(1.0)
    f = FSDP(m, wrap_cls=(nn.Linear,))
    opt = FusedShardedOptimizer(f.engine, "adamw", lr=1e-3) if fused else \
        ShardedOptimizer(torch.optim.AdamW(f.parameters(), lr=1e-3), f.engine)
    if not fused:      # a plain optimizer creates its state lazily: one throw-away step gives it its shape
        opt.zero_grad()
        f(torch.zeros(4, 256)).sum().backward()
        opt.step()
    dcp_io.load(f, opt, path)
    sd = f.state_dict()
    ref = torch.load(path + "/full_ref.pt")
    for k, v in ref.items():
        assert torch.equal(sd[k], v), k
    g = torch.Generator().manual_seed(99)
    opt.zero_grad()
    f(torch.randn(4, 256, generator=g)).sum().backward()
    opt.step()
    sd2 = f.state_dict()
    if rank == 0:
        torch.save(sd2, path + f"/after_{world}.pt")


def test_dcp_format_checkpoint_reshards_across_world_sizes(tmp_path):
    import os

    for fused in (True, False):
        path = str(tmp_path / f"dcp_{int(fused)}")
        os.makedirs(path)
        run_distributed(_dcp_save, world=2, args=(path, fused))
        files = sorted(os.listdir(path))
        assert ".metadata" in files and "__0_0.distcp" in files and "__1_0.distcp" in files, files
        for w in (2, 1, 3):
            run_distributed(_dcp_load, world=w, args=(path, fused))
        a2, a1, a3 = (torch.load(path + f"/after_{w}.pt") for w in (2, 1, 3))
        for k in a2:
            assert torch.allclose(a2[k], a1[k], atol=1e-6) and torch.allclose(a2[k], a3[k], atol=1e-6), k


def test_reference_reader_loads_flat_checkpoint_written_here(tmp_path):
    """The flat sharded files written by this package at world size 2 (with optimizer state) are read back by the
    reference's own ``ShardTensorUtil`` / ``ShardOptim`` (run in a clean interpreter whose only ``atorch`` is the
    unmodified reference installed under baseline/_ref)."""
    import os
    import subprocess
    import sys

    import pytest

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "atorch")):
        pytest.skip("the reference is not installed under baseline/_ref")
    path = str(tmp_path / "flat")
    run_distributed(_save, world=2, args=(path, False))
    script = r"""
import sys, torch
if not torch.cuda.is_available():      # the reader ends with a device synchronise; there is no device here
    torch.cuda.synchronize = lambda *a, **k: None
    torch.cuda.current_device = lambda: 0
from atorch.utils.fsdp_save_util import ShardTensorUtil
import atorch
assert "baseline/_ref" in atorch.__file__.replace("\\", "/"), atorch.__file__
path = sys.argv[1]
ref = torch.load(path + "/full_ref.pt")
util = ShardTensorUtil(path, 0, 1, device="cpu")
bad = []
for k, v in ref.items():
    t = util.load_tensor_by_name(k)
    if t is None or not torch.equal(t.reshape(v.shape).to(v.dtype), v):
        bad.append(k)
print("params", len(ref), "bad", bad)
assert not bad, bad
"""
    env = dict(os.environ, PYTHONPATH=ref)
    res = subprocess.run([sys.executable, "-c", script, path], cwd=str(tmp_path), env=env, capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "bad []" in res.stdout
