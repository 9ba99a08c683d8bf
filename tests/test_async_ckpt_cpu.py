"""Asynchronous flat checkpoints, tracker file, DCP-style manager, init-from-checkpoint (CPU)."""
import os

import torch
import torch.nn as nn

from tests.test_fsdp_cpu import make_mlp


def _sharded():
    from atorch_b200.parallel.fsdp import FSDP, FusedShardedOptimizer

    f = FSDP(make_mlp(), wrap_cls=(nn.Linear,))
    opt = FusedShardedOptimizer(f.engine, "adamw", lr=1e-2)
    f(torch.randn(4, 256)).sum().backward()
    opt.step()
    return f, opt


def test_async_save_tracker_and_load(tmp_path):
    from atorch_b200.trainer.fsdp import ExtraState, FsdpShardCkptAsyncSaver, FsdpShardDcpCkptLoader
    from atorch_b200.utils import fsdp_async_ckpt_util as A

    f, opt = _sharded()
    saver = FsdpShardCkptAsyncSaver()
    saver.save(7, str(tmp_path), module=f, optimizer=opt, extra_state=ExtraState(iteration=7, consumed_samples=28))
    saver.finish()
    assert A.latest_checkpoint_step(str(tmp_path)) == 7
    assert os.path.exists(tmp_path / "iter_0000007" / ".metadata")   # torch.distributed.checkpoint format
    ref = {k: v.clone() for k, v in f.state_dict().items()}
    f2, opt2 = _sharded()
    with torch.no_grad():
        f2.engine.master.add_(1.0)
    es = ExtraState()
    FsdpShardDcpCkptLoader().load(str(tmp_path), model=f2, optimizer=opt2, extra_state=es)
    assert es.iteration == 7 and es.consumed_samples == 28 and opt2.step_count == 1
    for k, v in f2.state_dict().items():
        assert torch.equal(v, ref[k])
    A.save_checkpoint(9, f, opt, str(tmp_path), storage_type=A.StorageType.MEMORY)
    assert 9 in A._WRITER.memory


def test_dcp_manager_and_init_fn(tmp_path):
    from atorch_b200.checkpoint.torch_checkpoint import TorchDCPCheckpointManager
    from atorch_b200.utils.fsdp_init_util import FSDPCkptConfig, FSDPInitFn

    f, opt = _sharded()
    mgr = TorchDCPCheckpointManager(str(tmp_path / "m"), interval=2, keep_latest_k=2)
    assert not mgr.save(1, f, opt)
    for s in (2, 4, 6):
        assert mgr.save(s, f, opt, train_state={"tokens": s * 10})
    assert mgr.steps() == [4, 6]
    f2, opt2 = _sharded()
    st = mgr.load(f2, opt2)
    assert st["step"] == 6 and st["tokens"] == 60
    plain = nn.Linear(4, 4)
    sched = torch.optim.lr_scheduler.StepLR(torch.optim.SGD(plain.parameters(), lr=1.0), 1)
    m2 = TorchDCPCheckpointManager(str(tmp_path / "p"))
    m2.save(1, plain, lr_scheduler=sched)
    assert m2.load(nn.Linear(4, 4))["step"] == 1
    # build a fresh model whose modules are filled from the flat checkpoint
    model = make_mlp()
    with torch.no_grad():
        for p in model.parameters():
            p.zero_()
    init = FSDPInitFn(model, 0, FSDPCkptConfig(flat_ckpt_path=str(tmp_path / "m" / "step-6")))
    for m in model.modules():
        if isinstance(m, nn.Linear):
            init(m)
    ref = f.state_dict()
    for k, v in model.state_dict().items():
        assert torch.equal(v, ref[k])
    assert not init.missing
