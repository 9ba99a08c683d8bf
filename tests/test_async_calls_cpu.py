"""Asynchronous calls with distributed finalisation (trainer/async_calls.py) on two gloo ranks: a call is finalised
only when it is done on every rank, finalisation runs in order and on all ranks, a failure or a timeout on one rank is
seen by all, and the checkpoint saver built on it writes its tracker last."""
import os
import time

import torch

from tests.dist_utils import run_distributed


def _write(path, rank, delay):
    time.sleep(delay)
    with open(os.path.join(path, f"part{rank}.bin"), "w") as f:
        f.write("x" * 10)


def _boom(rank):
    if rank == 1:
        raise RuntimeError("disk full")


def _sleep(seconds):
    time.sleep(seconds)


def _worker(rank, world, root, mode):
    import torch.distributed as dist

    from atorch_b200.trainer.async_calls import (AsyncCallsQueue, AsyncCheckpointSaver, AsyncRequest,
                                                 DistributedAsyncCaller)

    # 1. rank 1 is slower: nobody finalises before it is done; finalisers run in order on every rank
    q = AsyncCallsQueue(mode)
    log = []
    d0 = os.path.join(root, "a")
    os.makedirs(d0, exist_ok=True)
    req = AsyncRequest(_write, (d0, rank, 0.1 if rank == 0 else 1.0), [])
    req.add_finalize_fn(lambda: log.append("first"))
    req.add_finalize_fn(lambda: log.append("second"))
    idx = q.schedule_async_request(req)
    time.sleep(0.4)                                   # rank 0's own call is over, rank 1's is not
    assert q.maybe_finalize_async_calls(blocking=False) == [] and log == []
    assert q.get_num_unfinalized_calls() == 1
    assert q.maybe_finalize_async_calls(blocking=True) == [idx]
    assert log == ["first", "second"] and q.get_num_unfinalized_calls() == 0
    assert sorted(os.listdir(d0)) == ["part0.bin", "part1.bin"]
    try:
        q.calls  # frozen requests refuse new finalisers
        req.freeze().add_finalize_fn(lambda: None)
        raise AssertionError("a frozen request accepted a finaliser")
    except RuntimeError:
        pass

    # 2. a failure on one rank is reported on all, and its finalisers do not run
    ran = []
    bad = q.schedule_async_request(AsyncRequest(_boom, (rank,), [lambda: ran.append(1)]))
    assert q.maybe_finalize_async_calls(blocking=True) == [bad]
    assert q.failed == [bad] and ran == []

    # 3. a call that outlives its timeout is terminated and counts as failed everywhere (process mode only)
    if mode == "process":
        c = DistributedAsyncCaller("process", timeout=0.3)
        c.schedule_async_call(_sleep, (30.0 if rank == 0 else 0.0,))
        t0 = time.time()
        done, failed = c.is_current_async_call_done(blocking=True)
        assert done and failed and time.time() - t0 < 10

    # 4. the saver: tracker only after every rank has written
    saver = AsyncCheckpointSaver(os.path.join(root, "ckpt"), mode)
    d1 = os.path.join(root, "ckpt", "iter_0000007")
    os.makedirs(d1, exist_ok=True)
    dist.barrier()
    saver.save(7, _write, (d1, rank, 0.0 if rank == 0 else 0.8))
    time.sleep(0.3)
    saver.maybe_finalize()
    assert saver.latest_iteration() is None
    saver.close()
    dist.barrier()
    assert saver.latest_iteration() == 7 and sorted(os.listdir(d1)) == ["part0.bin", "part1.bin"]
    # synchronous execution of a request has the same effects
    out = []
    AsyncRequest(lambda: out.append("run"), (), [lambda: out.append("fin")]).execute_sync()
    assert out == ["run", "fin"]


def test_async_calls_process_mode(tmp_path):
    run_distributed(_worker, world=2, args=(str(tmp_path), "process"), timeout=120)


def test_async_calls_thread_mode(tmp_path):
    run_distributed(_worker, world=2, args=(str(tmp_path), "thread"), timeout=120)
