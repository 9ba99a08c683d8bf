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
