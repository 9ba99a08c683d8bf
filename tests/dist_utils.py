"""Helpers to run a function on N local ranks (gloo on CPU, nccl when GPUs are available)."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, backend, fn, args, err_q):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NPROC_PER_NODE=str(world), NODE_SIZE="1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    try:
        import atorch_b200

        torch.manual_seed(0)
        assert atorch_b200.init_distributed(backend, set_cuda_device_using_local_rank=(backend == "nccl"))
        fn(rank, world, *args)
        atorch_b200.reset_distributed()
    except Exception:
        err_q.put((rank, traceback.format_exc()))
        raise


def run_distributed(fn, world: int = 2, args=(), backend: str = "gloo", timeout: float = 120.0):
    """Spawn ``world`` processes running ``fn(rank, world, *args)``; raises if any rank fails."""
    ctx = mp.get_context("spawn")
    err_q = ctx.SimpleQueue()
    port = find_free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, backend, fn, args, err_q)) for r in range(world)]
    for p in procs:
        p.start()
    import time as _time

    deadline = _time.time() + timeout
    for p in procs:
        p.join(max(0.1, deadline - _time.time()))
    failed = []
    for r, p in enumerate(procs):
        if p.is_alive():
            p.kill()
            failed.append((r, "timeout"))
        elif p.exitcode != 0:
            failed.append((r, f"exit code {p.exitcode}"))
    msgs = []
    while not err_q.empty():
        msgs.append(err_q.get())
    if failed or msgs:
        raise AssertionError("distributed run failed: " + repr(failed) + "\n" + "\n".join(f"[rank {r}]\n{m}" for r, m in msgs))
