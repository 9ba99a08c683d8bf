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


_REF_WRITER = r"""
import os, sys, torch, torch.nn as nn, torch.distributed as dist, torch.multiprocessing as mp


def make_mlp():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(256, 512), nn.ReLU(), nn.Linear(512, 512), nn.ReLU(), nn.Linear(512, 512), nn.ReLU(),
                      nn.Linear(512, 10))
    for p in m.parameters():
        if p.dim() > 1:
            nn.init.normal_(p, std=0.02)
    return m


def run(rank, world, path, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.synchronize = lambda *a, **k: None      # the writer ends with a device synchronise; no device here
    torch.cuda.current_device = lambda: 0
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
    from torch.distributed.fsdp.wrap import ModuleWrapPolicy
    import atorch
    from atorch.utils.fsdp_save_util import save_fsdp_flat_param, save_fsdp_optim_param
    assert "baseline/_ref" in atorch.__file__.replace("\\", "/"), atorch.__file__
    f = FSDP(make_mlp(), auto_wrap_policy=ModuleWrapPolicy({nn.Linear}), use_orig_params=True,
             device_id=torch.device("cpu"))
    opt = torch.optim.AdamW(f.parameters(), lr=1e-3)
    g = torch.Generator().manual_seed(7 + rank)
    for _ in range(2):
        opt.zero_grad()
        f(torch.randn(4, 256, generator=g)).sum().backward()
        opt.step()
    save_fsdp_flat_param(f, path)
    save_fsdp_optim_param(f, opt, path)
    with FSDP.summon_full_params(f, writeback=False):
        full = {k.replace("_fsdp_wrapped_module.", ""): v.detach().clone() for k, v in f.named_parameters()}
    if rank == 0:
        torch.save(full, path + "/full_ref.pt")
        # the optimizer state to expect: the same two steps on an unsharded copy with the ranks' gradients averaged
        plain = make_mlp()
        popt = torch.optim.AdamW(plain.parameters(), lr=1e-3)
        gens = [torch.Generator().manual_seed(7 + r) for r in range(world)]
        for _ in range(2):
            popt.zero_grad()
            (sum(plain(torch.randn(4, 256, generator=g_)).sum() for g_ in gens) / world).backward()
            popt.step()
        torch.save({n: {k: v for k, v in popt.state[p_].items() if k != "step"} for n, p_ in plain.named_parameters()},
                   path + "/full_opt_ref.pt")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    os.makedirs(sys.argv[1], exist_ok=True)
    mp.spawn(run, args=(2, sys.argv[1], int(sys.argv[2])), nprocs=2)
"""


def _load_reference_ckpt(rank, world, path):
    from atorch_b200.parallel.fsdp import FSDP, ShardedOptimizer
    from atorch_b200.utils.fsdp_save_util import ShardOptim, load_fsdp_flat_param

    m = make_mlp()
    with torch.no_grad():
        for p in m.parameters():
            p.add_(1.0)
    f = FSDP(m, wrap_cls=(nn.Linear,))
    load_fsdp_flat_param(f, path)
    sd = f.state_dict()
    ref = torch.load(path + "/full_ref.pt")
    assert set(ref) == set(sd), (sorted(ref), sorted(sd))
    for k, v in ref.items():
        assert torch.equal(sd[k], v), k
    opt = ShardedOptimizer(torch.optim.AdamW(f.parameters(), lr=1e-3), f.engine)
    ShardOptim(path).load_into(f, opt)
    ref_opt = torch.load(path + "/full_opt_ref.pt")
    so = ShardOptim(path)
    for name, st in ref_opt.items():
        n = st["exp_avg"].numel()
        for key in ("exp_avg", "exp_avg_sq"):
            got = so.load_state_slice(name, key, 0, n)
            assert got is not None and torch.allclose(got, st[key].reshape(-1), rtol=1e-4, atol=1e-9), (name, key)


def test_flat_checkpoint_written_by_the_reference_loads_here(tmp_path):
    """The unmodified reference (torch FSDP on two gloo ranks, its own ``save_fsdp_flat_param`` /
    ``save_fsdp_optim_param``) writes a flat checkpoint; this package's loader restores it into its own sharded
    engine at world size 1 and 4: parameters bit-exact against the reference run's gathered parameters, optimizer
    state against the same two steps on an unsharded copy."""
    import os
    import subprocess
    import sys

    import pytest

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "atorch")):
        pytest.skip("the reference is not installed under baseline/_ref")
    path = str(tmp_path / "ref_flat")
    script = tmp_path / "ref_writer.py"
    script.write_text(_REF_WRITER)
    env = dict(os.environ, PYTHONPATH=ref)
    res = subprocess.run([sys.executable, str(script), path, "29643"], cwd=str(tmp_path), env=env, capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert os.path.exists(path + "/flat_param.00001-00002") and os.path.exists(path + "/optim_param.00000-00002")
    for w in (1, 4):
        run_distributed(_load_reference_ckpt, world=w, args=(path,))
