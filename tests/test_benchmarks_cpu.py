"""The benchmark scripts of the MoE and local-SGD configs run end to end on CPU with tiny models."""
import json

from tests.dist_utils import run_distributed


def _moe(rank, world):
    from atorch_b200.benchmarks import moe_bench

    moe_bench.main(["--tiny", "--fp8", "0", "--steps", "2", "--warmup", "1"])


def _lsgd(rank, world, H):
    from atorch_b200.benchmarks import local_sgd_bench

    local_sgd_bench.main(["--tiny", "--H", str(H), "--windows", "1"])


def test_moe_bench_tiny_expert_parallel():
    run_distributed(_moe, world=2, timeout=200)


def test_local_sgd_bench_tiny():
    run_distributed(_lsgd, world=2, args=(2,), timeout=200)
    run_distributed(_lsgd, world=2, args=(0,), timeout=200)


def _hybrid(rank, world, out):
    from atorch_b200.benchmarks import hybrid_bench

    losses = hybrid_bench.main(["--tiny", "--tp", "2", "--pp", "2", "--micro-batches", "4", "--steps", "4",
                                "--warmup", "0"])
    if losses:
        import torch

        torch.save(losses, f"{out}.{rank}")


def test_hybrid_tp_pp_dp_tiny(tmp_path):
    import glob

    import torch

    out = str(tmp_path / "l")
    run_distributed(_hybrid, world=8, args=(out,), timeout=300)
    files = glob.glob(out + ".*")
    assert files, "no last-stage rank reported losses"
    losses = torch.load(files[0])
    assert len(losses) == 4 and all(l == l for l in losses) and losses[-1] < losses[0], losses
