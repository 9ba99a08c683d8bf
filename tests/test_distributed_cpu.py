"""Process-group runtime on CPU/gloo: rank arithmetic, named groups, data partition, seq all-to-all."""
import torch
import torch.distributed as dist

from atorch_b200.distributed import distributed as D
from tests.dist_utils import run_distributed


def test_compute_group_ranks_matches_documented_layout():
    r = D.compute_group_ranks([("tensor", 4), ("pipeline", 2), ("data", 2)], list(range(16)))
    assert r["tensor"] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11], [12, 13, 14, 15]]
    assert r["pipeline"] == [[0, 4], [1, 5], [2, 6], [3, 7], [8, 12], [9, 13], [10, 14], [11, 15]]
    assert r["data"] == [[0, 8], [1, 9], [2, 10], [3, 11], [4, 12], [5, 13], [6, 14], [7, 15]]
    same = D.get_ranks_in_same_group(([("tensor", 2), ("data", 4)], None), my_rank=5, world=8)
    assert same == {"tensor": [4, 5], "data": [1, 3, 5, 7]}
    order = [3, 2, 1, 0]
    r2 = D.compute_group_ranks([("a", 2), ("b", 2)], order)
    assert r2["a"] == [[3, 2], [1, 0]] and r2["b"] == [[3, 1], [2, 0]]


def _groups(rank, world):
    D.create_parallel_group(([("tensor", 2), ("data", 2)], None))
    assert D.parallel_group_size("tensor") == 2 and D.parallel_group_size("data") == 2
    assert D.parallel_rank("tensor") == rank % 2 and D.parallel_rank("data") == rank // 2
    _, ranks = D.parallel_group_and_ranks("tensor")
    assert ranks == [rank - rank % 2, rank - rank % 2 + 1]
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=D.parallel_group("data"))
    assert t.item() == (rank % 2) * 2 + 2            # ranks r and r+2
    assert D.get_data_partition_rank_and_size() == (rank // 2, 2)
    with D.ParallelGroupContextManager("critic_"):
        D.create_parallel_group(([("data", world)], None))
        assert D.parallel_group_size("data") == world
        assert D.parallel_group("tensor") is None
    assert D.parallel_group_size("data") == 2
    D.destroy_parallel_group()
    D.create_parallel_group(([("zero", 2), ("data", 2)], None))
    assert D.get_data_partition_rank_and_size() == ((rank // 2) * 2 + rank % 2, 4)
    D.destroy_parallel_group()
    D.create_parallel_group(([("pipe", 2), ("data", 2)], None))
    assert D.is_pipe_first_stage() == (rank % 2 == 0) and D.is_pipe_last_stage() == (rank % 2 == 1)
    assert D.pipe_next_rank() == (rank + 1 if rank % 2 == 0 else rank - 1)


def test_named_groups_gloo():
    run_distributed(_groups, world=4)


def _seq_a2a(rank, world):
    D.create_sequence_parallel_group(world)
    assert D.get_sequence_parallel_size() == world and D.get_sequence_parallel_rank() == rank
    B, S_local, H, Dh = 2, 3, 4, 5
    full = torch.arange(B * S_local * world * H * Dh, dtype=torch.float32).view(B, S_local * world, H, Dh)
    mine = full[:, rank * S_local:(rank + 1) * S_local].clone().requires_grad_()
    out = D.seq_all_to_all(mine, 2, 1, D.get_sequence_parallel_group())     # scatter heads, gather sequence
    hpr = H // world
    assert torch.equal(out, full[:, :, rank * hpr:(rank + 1) * hpr])
    back = D.seq_all_to_all(out, 1, 2, D.get_sequence_parallel_group())
    assert torch.equal(back, mine)
    back.sum().backward()
    assert torch.equal(mine.grad, torch.ones_like(mine))


def test_seq_all_to_all_gloo():
    run_distributed(_seq_a2a, world=2)


def _mesh(rank, world):
    D.create_parallel_group(([("zero", 2), ("data", 2)], None, False, True))
    assert D.get_device_mesh("zero") is not None
    _, ranks = D.parallel_group_and_ranks("zero")
    assert ranks == [rank - rank % 2, rank - rank % 2 + 1]


def test_device_mesh_groups():
    run_distributed(_mesh, world=4)
