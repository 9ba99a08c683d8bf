"""Data utilities on CPU: preloader, unordered / batch-shuffled loaders, elastic shards, shared-memory loader."""
import multiprocessing as mp

import torch

from atorch_b200.data import (ElasticDataset, GpuPreLoader, ShardService, ShmDataloader, UnorderedDataLoader,
                              UnshuffledBatchDataLoader, expand_batch_dim, get_elastic_dataloader, get_sample_batch)


class DS(torch.utils.data.Dataset):
    def __len__(self):
        return 20

    def __getitem__(self, i):
        return {"x": torch.full((3,), float(i)), "i": i}


def test_preloader_and_utils():
    dl = torch.utils.data.DataLoader(DS(), batch_size=4)
    got = [b["i"].tolist() for b in GpuPreLoader(dl, device="cpu", post_processing=lambda b: b)]
    assert got == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11], [12, 13, 14, 15], [16, 17, 18, 19]]
    assert get_sample_batch(DS(), num=2)["x"].shape == (2, 3)
    assert expand_batch_dim({"a": torch.ones(3), "b": 2}, 4)["a"].shape == (4, 3)


def test_unordered_and_batch_shuffle():
    seen = sorted(i for b in UnorderedDataLoader(DS(), batch_size=4, num_workers=3) for i in b["i"].tolist())
    assert seen == list(range(20))
    dl = UnshuffledBatchDataLoader(DS(), batch_size=4, seed=1)
    batches = [b["i"].tolist() for b in dl]
    assert all(b == list(range(b[0], b[0] + 4)) for b in batches) and len(batches) == 5
    assert batches != sorted(batches)
    dl.set_epoch(1)
    assert [b["i"].tolist() for b in dl] != batches


def test_elastic_shards_recover():
    svc = ShardService(dataset_size=30, shard_size=10)
    t = svc.fetch(worker=0)
    assert t[1:] == (0, 10)
    assert svc.recover_worker(0) == 1          # worker 0 died: its shard goes back
    out = [int(x) for b in get_elastic_dataloader(lambda i: torch.tensor(i), 30, batch_size=5, service=svc, worker=1)
           for x in b]
    assert sorted(out) == list(range(30)) and svc.finished()


def _reader(q, prefix):
    dl = ShmDataloader(None, rank=1, group_size=2, shm_name_prefix=prefix, slot_bytes=1 << 16)
    q.put([b["i"].tolist() for b in dl])
    dl.close()


def test_shm_dataloader(tmp_path):
    prefix = f"atbtest_{abs(hash(str(tmp_path))) % 100000}_"
    master = ShmDataloader(DS(), {"batch_size": 5}, rank=0, group_size=2, shm_name_prefix=prefix, slot_bytes=1 << 16)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_reader, args=(q, prefix))
    p.start()
    mine = [b["i"].tolist() for b in master]
    theirs = q.get(timeout=60)
    p.join(30)
    master.close()
    assert mine == theirs and len(mine) == 4


def _square(x):
    return None if x == 5 else torch.tensor([x * x], dtype=torch.float32)


def _plus_one(i):
    return i + 1


def test_coworker_dataset_over_grpc_and_data_info_service():
    """Two coworker services on 127.0.0.1; percentage mode and rpc-worker mode give the same batches as local
    processing; failed samples are padded; the data-info directory hands out coworkers in arrival order."""
    import queue
    import threading

    from atorch_b200.data import build_coworker_dataloader
    from atorch_b200.service.coworker_data_service import create_coworker_rpc_service
    from atorch_b200.service.data_info_service import create_data_info_service
    from atorch_b200.service.rpc_clients import (CoworkerRpcClient, create_data_info_rpc_client,
                                                 create_gpu_pod_rpc_clients)

    q = queue.Queue()
    servers = [create_coworker_rpc_service(0, q), create_coworker_rpc_service(0, None)]
    for s in servers:
        s.start()
    addrs = [f"127.0.0.1:{s.bound_port}" for s in servers]
    try:
        assert CoworkerRpcClient(addrs[0]).ping()
        want = [[(i + 1) ** 2 for i in range(b, b + 4)] for b in range(0, 16, 4)]
        for kw in ({"coworker_process_percentage": 0.5}, {"num_rpc_workers": 1, "num_workers": 1}, {}):
            dl = build_coworker_dataloader(_square, 16, pre_process_fn=_plus_one, batch_size=4, shuffle=False,
                                           num_rpc_fuse=1, need_padding_for_none=True, coworker_addrs=addrs, **kw)
            got = [sorted(int(v) for v in b.view(-1)) for b in dl]
            for g, w in zip(got, want):
                w = [v for v in w if v != 25]          # sample 4 -> 5 fails and is replaced by a random other one
                assert all(v in g for v in w) and len(g) == 4, (kw, g, w)
        # pull model: a coworker queues finished batches and reports them; the trainer asks where to fetch
        info = create_data_info_service(0)
        info.start()
        q.put({"x": torch.ones(2)})
        create_gpu_pod_rpc_clients([f"127.0.0.1:{info.bound_port}"])[0].report_data_info(addrs[0], 1)
        where = create_data_info_rpc_client(f"127.0.0.1:{info.bound_port}").get_data_info()
        assert where == addrs[0]
        assert torch.equal(CoworkerRpcClient(where).get_batch_data()["x"], torch.ones(2))
        info.stop(None)
    finally:
        for s in servers:
            s.stop(None)
    del threading
